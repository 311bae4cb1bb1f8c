// Stand-in for the reference's llis/job/job.h, used ONLY to compile the reference's JobQueue class
// (include/llis/server/scheduler_full3.h:26-208) on its own: JobQueue reads nothing of a job except
// its type id and its priority.  Test infrastructure; never part of the product.
#pragma once
#include <cstdint>
#include <cstddef>
namespace llis {
using JobId = uint32_t;
using JobRefId = uint32_t;
namespace job {
class Job {
  public:
    Job(JobRefId type, double priority, uint64_t tag) : type_(type), priority_(priority), tag_(tag) {}
    JobRefId get_registered_job_id() const { return type_; }
    double get_priority() const { return priority_; }
    uint64_t tag() const { return tag_; }
  private:
    JobRefId type_;
    double priority_;
    uint64_t tag_;
};
}  // namespace job
}  // namespace llis
