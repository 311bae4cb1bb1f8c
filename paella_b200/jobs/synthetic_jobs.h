// Synthetic jobs of the scheduler stress configuration: vec_add and bounded spin kernels.
// Stage protocols follow jobs/vec_add_coroutine/vec_add_coroutine.cu:115-141 (H2D copy,
// N x vec_add, D2H copy with pre-notify) and jobs/dummy_short/dummy_short.cu:43-62
// (N compute stages, pre-notify on the last).
#pragma once

#include <cuda_runtime.h>
#include <llis/job/context.h>
#include <llis/job/job.h>

#include <cstdlib>

#include "paella_b200.h"

namespace pbjobs {

inline unsigned long env_ul(const char* name, unsigned long dflt) {
    const char* v = std::getenv(name);
    return (v && *v) ? std::strtoul(v, nullptr, 0) : dflt;
}

// out[i] += in[i] over n floats (PB_VEC_ADD_N, default 2^20), `iters` launches per job.
class VecAddJob : public llis::job::Job {
  public:
    VecAddJob() : n_(env_ul("PB_VEC_ADD_N", 1ul << 20)), iters_((int)env_ul("PB_VEC_ADD_ITERS", 10)) {}
    size_t get_input_size() override { return n_ * sizeof(float); }
    size_t get_output_size() override { return n_ * sizeof(float); }
    size_t get_param_size() override { return 4; }
    void full_init(void* io_ptr) override {
        if (cudaMalloc(&in_dev_, n_ * sizeof(float)) != cudaSuccess || cudaMalloc(&out_dev_, n_ * sizeof(float)) != cudaSuccess ||
            cudaMemset(out_dev_, 0, n_ * sizeof(float)) != cudaSuccess) { set_error(PB_ERR_CUDA); return; }
        pb_launch_info li;
        pb_vec_add_info(n_, &li);
        decl_.num_blocks = li.num_blocks;
        decl_.num_threads_per_block = li.threads_per_block;
        decl_.num_registers_per_thread = li.regs_per_thread;
        init(io_ptr);
    }
    void init(void* io_ptr) override {
        io_ = static_cast<char*>(io_ptr);
        next_ = 0;
        resident_ = llis::job::Context::device_resident();
        set_is_mem();
    }
    void run_next() override {
        cudaStream_t st = get_cuda_stream();
        if (next_ == 0) {
            if (!resident_ && cudaMemcpyAsync(in_dev_, io_, n_ * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess) set_error(PB_ERR_CUDA);
        } else if (next_ <= iters_) {
            if (pb_vec_add_launch((float*)out_dev_, (const float*)in_dev_, n_, st, get_id(), get_finished_block_notifier()) != PB_OK) set_error(PB_ERR_CUDA);
        } else {
            if (!resident_ && cudaMemcpyAsync(io_ + get_output_offset(), out_dev_, n_ * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess) set_error(PB_ERR_CUDA);
        }
        ++next_;
        if (next_ <= iters_) { unset_is_mem(); set_next_stage(decl_); }
        else if (next_ == iters_ + 1) { set_is_mem(); set_pre_notify(); }
    }
    bool has_next() const override { return next_ < iters_ + 2; }

  private:
    size_t n_;
    int iters_;
    void* in_dev_ = nullptr;
    void* out_dev_ = nullptr;
    char* io_ = nullptr;
    int next_ = 0;
    bool resident_ = false;
    llis::job::StageDecl decl_;
};

// `kernels` launches of a grid that holds its SM slots for spin_ns per block.
class SpinJob : public llis::job::Job {
  public:
    SpinJob(unsigned kernels, unsigned long spin_ns, const char* blocks_env)
        : kernels_((int)kernels), spin_ns_(spin_ns), blocks_((unsigned)env_ul(blocks_env, 148)) {}
    size_t get_input_size() override { return 5; }
    size_t get_output_size() override { return 11; }
    size_t get_param_size() override { return 4; }
    void full_init(void* io_ptr) override {
        pb_launch_info li;
        pb_spin_info(blocks_, &li);
        decl_.num_blocks = li.num_blocks;
        decl_.num_threads_per_block = li.threads_per_block;
        decl_.num_registers_per_thread = li.regs_per_thread;
        init(io_ptr);
    }
    void init(void*) override {
        next_ = 0;
        unset_is_mem();
        set_next_stage(decl_);
        if (kernels_ == 1) set_pre_notify();
    }
    void run_next() override {
        if (pb_spin_launch(blocks_, spin_ns_, nullptr, get_cuda_stream(), get_id(), get_finished_block_notifier()) != PB_OK) set_error(PB_ERR_CUDA);
        ++next_;
        if (next_ == kernels_ - 1) set_pre_notify();
    }
    bool has_next() const override { return next_ < kernels_; }

  private:
    int kernels_;
    unsigned long spin_ns_;
    unsigned blocks_;
    int next_ = 0;
    llis::job::StageDecl decl_;
};

}  // namespace pbjobs
