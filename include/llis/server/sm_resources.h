// Whole-GPU occupancy tracker used by the kernel-level scheduler.
//
// Same model as the reference's SmResources (src/server/sm_resources.cpp:17-66,
// include/llis/server/sm_resources.h:25-31): an aggregate over all SMs of registers,
// shared memory, threads and block slots; acquire/release per batch of blocks of the
// stage in flight; job_fits tests the declared next stage against what is left.
// Added for Blackwell: tensor-memory columns (512 per SM) as a fifth component, and
// the totals are read from the device the server runs on (the reference reads device 0).
#pragma once

#include <llis/job/job.h>

namespace llis {
namespace server {

struct SmTotals {
    int regs = 0, smem = 0, threads = 0, blocks = 0, tmem_cols = 0;
    int num_sms = 0;
};

class SmResources {
  public:
    SmResources() = default;
    explicit SmResources(const SmTotals& t) : left_(t), max_(t) {}

    // Fills totals from cudaGetDeviceProperties(device); returns a pb_status.
    static int query_device(int device, SmTotals* out);

    void acquire(const job::Job* job, int num) { apply(job->cur_stage_decl(), -num); }
    void release(const job::Job* job, int num) { apply(job->cur_stage_decl(), num); }

    bool job_fits(const job::Job* job) const {
        const job::StageDecl& d = job->next_stage();
        const int nb = (int)d.num_blocks;
        return left_.regs >= (int)d.num_registers_per_thread * (int)d.num_threads_per_block * nb &&
               left_.smem >= (int)d.smem_size_per_block * nb && left_.threads >= (int)d.num_threads_per_block * nb &&
               left_.blocks >= nb && left_.tmem_cols >= (int)d.tmem_cols_per_block * nb;
    }
    bool is_full() const { return left_.regs <= 0 || left_.smem <= 0 || left_.threads <= 0 || left_.blocks <= 0; }
    // Nothing is acquired: no kernel stage is in flight.
    bool idle() const {
        return left_.regs == max_.regs && left_.smem == max_.smem && left_.threads == max_.threads && left_.blocks == max_.blocks &&
               left_.tmem_cols == max_.tmem_cols;
    }
    const SmTotals& left() const { return left_; }
    const SmTotals& total() const { return max_; }
    double occupancy() const;

  private:
    void apply(const job::StageDecl& d, int num) {
        left_.regs += (int)(d.num_registers_per_thread * d.num_threads_per_block) * num;
        left_.threads += (int)d.num_threads_per_block * num;
        left_.smem += (int)d.smem_size_per_block * num;
        left_.blocks += num;
        left_.tmem_cols += (int)d.tmem_cols_per_block * num;
    }
    SmTotals left_, max_;
};

}  // namespace server
}  // namespace llis
