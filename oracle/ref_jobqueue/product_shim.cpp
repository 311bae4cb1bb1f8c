// The same C entry points as ref_shim.cpp around the PRODUCT's ready queue (include/llis/server/job_queue.h),
// so that one fuzz test drives both.  Test infrastructure.
#include <llis/server/job_queue.h>

#include <cstdint>
#include <deque>

namespace {
class TagJob : public llis::job::Job {
  public:
    explicit TagJob(uint64_t tag) : tag_(tag) {}
    size_t get_input_size() override { return 0; }
    size_t get_output_size() override { return 0; }
    size_t get_param_size() override { return 0; }
    void full_init(void*) override {}
    void init(void*) override {}
    void run_next() override {}
    bool has_next() const override { return false; }
    uint64_t tag() const { return tag_; }
  private:
    uint64_t tag_;
};
struct Handle {
    explicit Handle(double threshold) : q(threshold) {}
    llis::server::JobQueue q;
    std::deque<TagJob> jobs;
};
}  // namespace

#define JQ_API __attribute__((visibility("default")))
extern "C" {
JQ_API void* jq_create(double unfairness_threshold) { return new Handle(unfairness_threshold); }
JQ_API void jq_destroy(void* h) { delete static_cast<Handle*>(h); }
JQ_API void jq_push(void* h, uint32_t type, double priority, uint64_t tag) {
    Handle* s = static_cast<Handle*>(h);
    s->jobs.emplace_back(tag);
    TagJob* j = &s->jobs.back();
    j->set_client_details(0, type);
    j->set_priority(priority);
    s->q.push(j);
}
JQ_API uint64_t jq_top(void* h) { return static_cast<TagJob*>(static_cast<Handle*>(h)->q.top())->tag(); }
JQ_API uint64_t jq_pop(void* h) { return static_cast<TagJob*>(static_cast<Handle*>(h)->q.pop())->tag(); }
JQ_API uint64_t jq_size(void* h) { return static_cast<Handle*>(h)->q.size(); }
}
