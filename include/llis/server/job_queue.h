// Ready queue of the kernel-level scheduler: highest priority first, with a
// deficit-counter fairness override between job types.
//
// Observable behaviour is that of the reference's JobQueue
// (include/llis/server/scheduler_full3.h:26-208): top()/pop() return the globally
// highest-priority job unless the type with the largest deficit counter has reached the
// unfairness threshold, in which case that type's best job goes first; every pop lowers
// the new-type deficit and the threshold by 1/num_types and the popped type's counter by
// 1; a type whose last job is popped forgets its counter; ties (equal priority, equal
// deficit) resolve by insertion order.
//
// Structure differs.  The reference keeps three std::multimaps with cross iterators
// (three red-black-tree updates per push and per pop).  Here each type owns one binary
// heap ordered by (priority desc, push sequence asc); the global top is the best of the
// per-type tops (a scan over at most a handful of types), and the type order is a scan
// over (deficit desc, activation sequence asc).  One heap operation per push/pop.
#pragma once

#include <algorithm>
#include <cfloat>
#include <cstdint>
#include <vector>

#include <llis/job/job.h>

namespace llis {
namespace server {

class JobQueue {
  public:
    explicit JobQueue(double unfairness_threshold) : unfairness_threshold_(unfairness_threshold) {}

    void push(job::Job* job) {
        const JobRefId type = job->get_registered_job_id();
        if (type >= types_.size()) types_.resize(type + 1);
        Type& t = types_[type];
        if (!t.known) {                      // new type, or one that forgot its counter
            t.known = true;
            t.deficit = new_type_deficit_;
            ++num_types_;
        }
        if (t.heap.empty()) t.active_seq = next_seq_++;   // (re)enters the type order behind equal deficits
        t.heap.push_back(Entry{job->get_priority(), next_seq_++, job});
        std::push_heap(t.heap.begin(), t.heap.end(), worse);
        ++size_;
    }

    job::Job* top() const { return types_[pick_type()].heap.front().job; }

    job::Job* pop() { return pop_of(pick_type()); }

    // Gang formation: takes the best queued job of `type` if `accept` says so, with the same counter
    // arithmetic as a pop(); NULL (nothing changed) when the type has no queued job or its best is refused.
    template <typename Pred>
    job::Job* pop_of_type_if(JobRefId type, Pred accept) {
        if (type >= types_.size() || types_[type].heap.empty() || !accept(types_[type].heap.front().job)) return nullptr;
        return pop_of(type);
    }

    bool empty() const { return size_ == 0; }
    size_t size() const { return size_; }
    double unfairness_threshold() const { return unfairness_threshold_; }

  private:
    job::Job* pop_of(size_t ti) {
        Type& t = types_[ti];
        std::pop_heap(t.heap.begin(), t.heap.end(), worse);
        job::Job* job = t.heap.back().job;
        t.heap.pop_back();
        --size_;

        const double fair_share = 1. / (double)num_types_;
        new_type_deficit_ -= fair_share;
        unfairness_threshold_ -= fair_share;
        if (t.heap.empty()) {
            t.known = false;                 // counter is reset when no job of the type is queued
            --num_types_;
        } else {
            t.deficit -= 1.;
            t.active_seq = next_seq_++;      // re-inserted behind types of equal deficit
        }
        if (new_type_deficit_ < 10. - DBL_MAX) rebase();
        return job;
    }

    struct Entry {
        double priority;
        uint64_t seq;
        job::Job* job;
    };
    struct Type {
        bool known = false;
        double deficit = 0;
        uint64_t active_seq = 0;
        std::vector<Entry> heap;
    };
    // heap comparator: a is worse than b
    static bool worse(const Entry& a, const Entry& b) {
        return a.priority < b.priority || (a.priority == b.priority && a.seq > b.seq);
    }

    size_t pick_type() const {
        // type with the largest deficit among those that have queued jobs
        size_t fair = SIZE_MAX, best = SIZE_MAX;
        for (size_t i = 0; i < types_.size(); ++i) {
            const Type& t = types_[i];
            if (t.heap.empty()) continue;
            if (fair == SIZE_MAX || t.deficit > types_[fair].deficit ||
                (t.deficit == types_[fair].deficit && t.active_seq < types_[fair].active_seq))
                fair = i;
            if (best == SIZE_MAX || worse(types_[best].heap.front(), t.heap.front())) best = i;
        }
        return types_[fair].deficit >= unfairness_threshold_ ? fair : best;
    }

    // Keeps the counters away from -DBL_MAX (reference: rebuild_type_map, scheduler_full3.h:135-140,163-185).
    void rebase() {
        for (Type& t : types_)
            if (t.known) t.deficit -= new_type_deficit_;
        unfairness_threshold_ -= new_type_deficit_;
        new_type_deficit_ = 0;
    }

    double unfairness_threshold_;
    double new_type_deficit_ = 0;
    unsigned num_types_ = 0;
    uint64_t next_seq_ = 0;
    size_t size_ = 0;
    std::vector<Type> types_;
};

}  // namespace server
}  // namespace llis
