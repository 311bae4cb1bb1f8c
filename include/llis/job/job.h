// The job plugin interface: what a libjob_*.so hands to the server through
// `extern "C" llis::job::Job* init_job()`.
//
// Drop-in for the reference's include/llis/job/job.h:16-336.  The seven virtuals
// keep their order (job.h:18-24) and every accessor the scheduler or a plugin uses
// keeps its name and meaning.  A job is a resumable sequence of stages; before each
// run_next() the scheduler reads the DECLARED resources of the next stage
// (blocks / threads / shared memory / registers, is_mem, is_pre_notify), and
// set_running() snapshots them as cur_* for the stage in flight.
//
// Deliberate differences:
//  * the per-SM prediction array hard-wired to 40 SMs (job.h:247,314) is gone; the
//    scheduler tracks whole-GPU aggregates read from the device properties;
//  * a stage may declare tensor-memory columns per block (set_tmem_cols_per_block),
//    a Blackwell resource the occupancy tracker needs for tcgen05 kernels;
//  * stage start times come from an injectable clock (set_stage_start_time_us) so
//    that a recorded trace replays to bit-identical priorities;
//  * an error flag (set_error / has_error): run_next() is void in the reference and
//    failures abort the process; here a plugin records the failure and the server
//    reports it to the client;
//  * a stage index beyond the admission-time length table contributes 0 to the
//    remaining-length decrement (the reference reads past the end, job.h:288-292).
//  * gangs: a plugin may state that up to `capacity` of its jobs can run as ONE launch per
//    stage (set_gang_decls); a scheduler that forms gangs dispatches the leader's stages
//    with the followers listed in Context, and declares for it the resources of a gang of
//    that size (apply_gang_size).  A job that never calls set_gang_decls has capacity 1 and
//    is scheduled exactly as in the reference.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include <llis/ipc/defs.h>
#include <llis/utils/align.h>

typedef struct CUstream_st* cudaStream_t;

namespace llis {
namespace job {

class FinishedBlockNotifier;

// Resources one stage asks for; the 4-vector of the reference plus TMEM columns.
struct StageDecl {
    unsigned num_blocks = 0;
    unsigned num_threads_per_block = 0;
    unsigned smem_size_per_block = 0;
    unsigned num_registers_per_thread = 0;
    unsigned tmem_cols_per_block = 0;
};

class Job {
  public:
    virtual size_t get_input_size() = 0;
    virtual size_t get_output_size() = 0;
    virtual size_t get_param_size() = 0;
    virtual void full_init(void* io_ptr) = 0;
    virtual void init(void* io_ptr) = 0;
    virtual void run_next() = 0;
    virtual bool has_next() const = 0;

    // ---- pinned I/O slot layout (job.h:54-60) -------------------------------
    size_t get_output_offset() { return utils::next_aligned_pos(get_input_size(), 8); }
    size_t get_pinned_mem_size() { return get_output_offset() + utils::next_aligned_pos(get_output_size(), 8); }

    // ---- identity -----------------------------------------------------------
    void set_id(JobId id) { id_ = id; unique_id_ = next_unique_id()++; }
    JobId get_id() const { return id_; }
    JobId get_unique_id() const { return unique_id_; }
    void set_client_details(ClientId client_id, JobRefId registered_job_id) {
        client_id_ = client_id;
        registered_job_id_ = registered_job_id;
    }
    ClientId get_client_id() const { return client_id_; }
    JobRefId get_registered_job_id() const { return registered_job_id_; }
    void* get_remote_ptr() const { return remote_ptr_; }
    void set_remote_ptr(void* p) { remote_ptr_ = p; }

    // ---- declaration of the NEXT stage (written by the plugin) ------------
    void set_num_blocks(unsigned v) { next_.num_blocks = v; }
    void set_num_threads_per_block(unsigned v) { next_.num_threads_per_block = v; }
    void set_smem_size_per_block(unsigned v) { next_.smem_size_per_block = v; }
    void set_num_registers_per_thread(unsigned v) { next_.num_registers_per_thread = v; }
    void set_tmem_cols_per_block(unsigned v) { next_.tmem_cols_per_block = v; }
    void set_next_stage(const StageDecl& d) { next_ = d; }
    unsigned get_num_blocks() const { return next_.num_blocks; }
    unsigned get_num_threads_per_block() const { return next_.num_threads_per_block; }
    unsigned get_smem_size_per_block() const { return next_.smem_size_per_block; }
    unsigned get_num_registers_per_thread() const { return next_.num_registers_per_thread; }
    unsigned get_tmem_cols_per_block() const { return next_.tmem_cols_per_block; }
    const StageDecl& next_stage() const { return next_; }

    bool is_mem() const { return is_mem_; }
    void set_is_mem() { is_mem_ = true; }
    void unset_is_mem() { is_mem_ = false; }
    bool is_pre_notify() const { return is_pre_notify_; }
    void set_pre_notify() { is_pre_notify_ = true; }
    void unset_pre_notify() { is_pre_notify_ = false; }

    // ---- the stage in flight (snapshot taken by set_running) --------------
    unsigned get_cur_num_blocks() const { return cur_.num_blocks; }
    unsigned get_cur_num_threads_per_block() const { return cur_.num_threads_per_block; }
    unsigned get_cur_smem_size_per_block() const { return cur_.smem_size_per_block; }
    unsigned get_cur_num_registers_per_thread() const { return cur_.num_registers_per_thread; }
    unsigned get_cur_tmem_cols_per_block() const { return cur_.tmem_cols_per_block; }
    const StageDecl& cur_stage_decl() const { return cur_; }
    int get_cur_stage() const { return cur_stage_; }

    // job.h:138-153.  `now_us` replaces the steady_clock read taken there.
    void set_running(cudaStream_t stream, double now_us) {
        is_running_ = true;
        cuda_stream_ = stream;
        num_running_blocks_ = (int)next_.num_blocks;
        num_pending_blocks_ = (int)next_.num_blocks;
        cur_ = next_;
        cur_is_mem_ = is_mem_;
        stage_start_time_us_ = now_us;
        ++cur_stage_;
    }
    bool is_running() const { return is_running_; }
    void unset_running() { is_running_ = false; }
    double get_stage_start_time_us() const { return stage_start_time_us_; }
    cudaStream_t get_cuda_stream() const { return cuda_stream_; }

    // Returns true while blocks of the stage are still to start (job.h:167-173).
    bool mark_block_start(unsigned num = 1) { return (num_pending_blocks_ -= (int)num) != 0; }
    // job.h:175-187: the stage stops running when every block has ended.
    void mark_block_finish(unsigned num = 1) {
        num_running_blocks_ -= (int)num;
        if (num_running_blocks_ <= 0) unset_running();
    }

    // Blocks of the stage in flight that have not ended yet / whether that stage is a copy (watchdog).
    unsigned running_blocks() const { return num_running_blocks_ > 0 ? (unsigned)num_running_blocks_ : 0u; }
    bool is_mem_stage_in_flight() const { return cur_is_mem_; }

    void set_finished_block_notifier(FinishedBlockNotifier* n) { finished_block_notifier_ = n; }
    FinishedBlockNotifier* get_finished_block_notifier() { return finished_block_notifier_; }

    // ---- scheduler bookkeeping ----------------------------------------------
    void set_started() { has_started_ = true; }
    void unset_started() { has_started_ = false; }
    bool has_started() const { return has_started_; }
    void set_priority(double p) { priority_ = p; }
    double get_priority() const { return priority_; }
    bool is_unfit() const { return is_unfit_; }
    void set_unfit() { is_unfit_ = true; }
    void unset_unfit() { is_unfit_ = false; }
    void inc_deficit_counter(float v) { deficit_counter_ += v; }
    float get_deficit_counter() const { return deficit_counter_; }

    // Remaining "length x resource" bookkeeping (job.h:278-292).  As in the reference
    // the job keeps the type's tables AS THEY WERE AT ADMISSION (later EWMA updates of
    // the type do not change this job's decrements); the copy lands in vectors whose
    // capacity survives instance reuse, so it allocates only on an instance's first
    // launches.  A stage beyond the snapshot contributes 0, where the reference
    // indexes past the end of its copy.
    void set_stage_lengths_resources(double total, const std::vector<double>& lengths, const std::vector<float>& resources) {
        cur_rl_ = total;
        stage_lengths_.assign(lengths.begin(), lengths.end());
        stage_resources_.assign(resources.begin(), resources.end());
    }
    double get_cur_rl() const { return cur_rl_; }
    void dec_cur_rl() {
        const size_t i = (size_t)(cur_stage_ + 1);
        if (i < stage_lengths_.size() && i < stage_resources_.size()) cur_rl_ -= stage_lengths_[i] * (double)stage_resources_[i];
    }

    // ---- gangs ------------------------------------------------------------------
    // Plugin: `row[n - 1]` is the declaration of the NEXT stage when it runs for a gang of n jobs
    // (n = 1 .. capacity); the row must stay valid until the next call.  Called by the plugin each
    // time it declares a stage (NULL / 1 = this stage runs one job per launch).
    void set_gang_decls(const StageDecl* row, unsigned capacity) { gang_row_ = row; gang_capacity_ = row ? capacity : 1; }
    unsigned get_gang_capacity() const { return gang_row_ ? gang_capacity_ : 1; }
    // Scheduler: the next stage will run for a gang of n (<= capacity) jobs led by this one.
    void apply_gang_size(unsigned n) { if (gang_row_ && n >= 1 && n <= gang_capacity_) next_ = gang_row_[n - 1]; }

    // ---- error reporting ------------------------------------------------------
    void set_error(int code) { if (!error_) error_ = code; }
    int has_error() const { return error_; }

    // Called before an instance is reused (job.h:26-34).
    void reset_internal() {
        unset_running();
        unset_started();
        unset_is_mem();
        unset_pre_notify();
        deficit_counter_ = 0;
        cur_stage_ = -1;
        unset_unfit();
        error_ = 0;
        gang_row_ = nullptr;
        gang_capacity_ = 1;
    }

  private:
    static unsigned& next_unique_id() { static unsigned c = 0; return c; }

    StageDecl next_;
    StageDecl cur_;
    bool is_mem_ = false;
    bool is_pre_notify_ = false;
    bool cur_is_mem_ = false;
    bool is_running_ = false;
    bool has_started_ = false;
    bool is_unfit_ = false;
    int cur_stage_ = -1;
    int error_ = 0;
    int num_running_blocks_ = 0;
    int num_pending_blocks_ = 0;
    cudaStream_t cuda_stream_ = nullptr;
    FinishedBlockNotifier* finished_block_notifier_ = nullptr;
    float deficit_counter_ = 0;
    double priority_ = 0;
    double cur_rl_ = 0;
    double stage_start_time_us_ = 0;
    std::vector<double> stage_lengths_;
    std::vector<float> stage_resources_;
    ClientId client_id_ = 0;
    JobRefId registered_job_id_ = 0;
    void* remote_ptr_ = nullptr;
    JobId id_ = 0;
    JobId unique_id_ = 0;
    const StageDecl* gang_row_ = nullptr;
    unsigned gang_capacity_ = 1;
};

}  // namespace job
}  // namespace llis
