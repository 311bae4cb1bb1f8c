// C entry points around the reference's own JobQueue class, compiled from the reference's header where it
// lies (include/llis/server/scheduler_full3.h:26-208) with the stand-in headers in stubs/.  The fuzz test
// drives this and the Python restatement (oracle/scheduler.py:RefJobQueue) and the product's JobQueue with
// the same push/pop sequences.  Test infrastructure; never linked into the product.
#include <llis/server/scheduler_full3.h>

#include <cstdint>
#include <deque>

namespace {
struct Handle {
    explicit Handle(double threshold) : q(threshold) {}
    llis::server::JobQueue q;
    std::deque<llis::job::Job> jobs;   // stable addresses
};
}  // namespace

#define JQ_API __attribute__((visibility("default")))
extern "C" {
JQ_API void* jq_create(double unfairness_threshold) { return new Handle(unfairness_threshold); }
JQ_API void jq_destroy(void* h) { delete static_cast<Handle*>(h); }
JQ_API void jq_push(void* h, uint32_t type, double priority, uint64_t tag) {
    Handle* s = static_cast<Handle*>(h);
    s->jobs.emplace_back(type, priority, tag);
    s->q.push(&s->jobs.back());
}
JQ_API uint64_t jq_top(void* h) { return static_cast<Handle*>(h)->q.top()->tag(); }
JQ_API uint64_t jq_pop(void* h) { return static_cast<Handle*>(h)->q.pop()->tag(); }
JQ_API uint64_t jq_size(void* h) { return static_cast<Handle*>(h)->q.size(); }
}
