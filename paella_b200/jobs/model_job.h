// Job adapter for a packed model.  Stage protocol of the reference's TVM adapters
// (jobs/tvm_mnist/tvm_mnist.cpp:35-47): init() leaves the job before its first stage with that
// stage declared; each run_next() enqueues exactly one operation on the job's stream and declares
// the resources of the next stage; the last stage carries pre-notify.  A stage here is one GROUP of
// the model's kernels (one CUDA-graph launch), and by default the request's pinned slot is read and
// written by the kernels themselves; PB_COPY_STAGES=1 restores the reference's H2D / D2H copy stages
// and PB_STAGE_GROUP=1 its one-kernel-per-stage granularity.  Written as a stage-index state machine instead of a
// boost coroutine; the server only sees the llis::job::Job interface.
//
// Gangs: when the server allows it (Context::max_gang() > 1) the adapter sizes its instance for that many
// images and tells the scheduler, per stage, what a gang of n such jobs declares; the scheduler may then
// dispatch this job as the LEADER of up to n - 1 queued jobs of the same model (listed in Context), and
// each run_next() enqueues the stage once for all of them: one batched launch, every member's input read
// from and result written to its own pinned slot.
//
// Differences from the reference adapters: the D2H stage copies the OUTPUT tensor (there
// it copies from the input buffer, tvm_mnist.cpp:46); the device comes from the server
// thread's context instead of being hard-wired to 0; CUDA failures set the job's error
// flag instead of being ignored.
#pragma once

#include <cuda_runtime.h>
#include <llis/job/context.h>
#include <llis/job/job.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "paella_b200.h"

namespace pbjobs {

class ModelJob : public llis::job::Job {
  public:
    ModelJob(const char* model_name, size_t in_floats, size_t out_floats)
        : name_(model_name), in_bytes_(in_floats * sizeof(float)), out_bytes_(out_floats * sizeof(float)) {}

    size_t get_input_size() override { return in_bytes_; }
    size_t get_output_size() override { return out_bytes_; }
    size_t get_param_size() override { return 4; }

    void full_init(void* io_ptr) override {
        const int device = llis::job::Context::get_device();
        const char* dir = std::getenv("LLIS_MODELS_DIR");
        const std::string path = std::string(dir ? dir : ".") + "/" + name_ + "-b200-pack.bin";
        pb_model* model = shared_model(device, path);
        if (!model) { set_error(PB_ERR_IO); return; }
        if (pb_model_input_bytes(model) != in_bytes_ || pb_model_output_bytes(model) != out_bytes_) { set_error(PB_ERR_INVALID); return; }
        // PB_COPY_STAGES=1: the reference's protocol (H2D copy stage, kernels, D2H copy stage).  Default:
        // the first kernel reads the pinned request slot and the last writes the result into it, so a
        // request is nothing but its kernel stages.
        const char* cs = std::getenv("PB_COPY_STAGES");
        copy_stages_ = cs && cs[0] == '1';
        cap_ = copy_stages_ ? 1 : (int)llis::job::Context::max_gang();
        if (cap_ > PB_MAX_GANG) cap_ = PB_MAX_GANG;
        if (cap_ < 1) cap_ = 1;
        // every gang size is prepared now (descriptors, graphs): nothing is built on the serving path
        if (pb_instance_create_batched(model, cap_, 1, &inst_) != PB_OK) { set_error(PB_ERR_CUDA); return; }
        remember(llis::job::Context::get_owner(), inst_);
        const int n = pb_model_num_groups(model);
        decls_.resize((size_t)n * (size_t)cap_);          // [group][gang size - 1]
        for (int i = 0; i < n; ++i)
            for (int nb = 1; nb <= cap_; ++nb) {
                pb_launch_info li;
                if (pb_model_group_info_batched(model, i, nb, &li) != PB_OK) { set_error(PB_ERR_INVALID); return; }
                llis::job::StageDecl& d = decls_[(size_t)i * cap_ + (nb - 1)];
                d.num_blocks = li.num_blocks;
                d.num_threads_per_block = li.threads_per_block;
                d.smem_size_per_block = li.smem_per_block;
                d.num_registers_per_thread = li.regs_per_thread;
                d.tmem_cols_per_block = li.tmem_cols_per_block;
            }
        num_groups_ = n;
        init(io_ptr);
    }

    void init(void* io_ptr) override {
        io_ptr_ = static_cast<char*>(io_ptr);
        next_ = 0;
        gang_n_ = 1;
        resident_ = llis::job::Context::device_resident();
        declare();
    }

    // Stage list: [H2D copy] group 0 .. group n-1 [D2H copy]; the copies exist only with PB_COPY_STAGES=1.
    void run_next() override {
        const int n = num_groups_;
        const int lead = copy_stages_ ? 1 : 0;
        cudaStream_t st = get_cuda_stream();
        const int cur = next_++;
        // the members of this dispatch: this job and, when it leads a gang, the followers the scheduler lists
        unsigned n_follow = 0;
        llis::job::Job* const* follow = llis::job::Context::get_gang(&n_follow);
        if ((int)n_follow + 1 > cap_) { set_error(PB_ERR_INVALID); n_follow = 0; }
        gang_n_ = 1 + (int)n_follow;       // a gang stays together: the following stages are declared for it
        declare();      // the stage that follows is declared before this one is enqueued
        if (!inst_) return;
        if (cur < lead) {
            if (!resident_) check(cudaMemcpyAsync(pb_instance_input_dev(inst_), io_ptr_, in_bytes_, cudaMemcpyHostToDevice, st));
        } else if (cur < lead + n) {
            const bool direct_io = !copy_stages_ && !resident_;
            const void* ins[PB_MAX_GANG];
            void* outs[PB_MAX_GANG];
            for (int i = 0; i < gang_n_; ++i) {
                char* io = i == 0 ? io_ptr_ : static_cast<ModelJob*>(follow[i - 1])->io_ptr_;     // followers are jobs of this type
                ins[i] = direct_io ? io : nullptr;
                // Loads issued by SMs keep few PCIe reads in flight (about 11 GB/s measured); a copy engine
                // streams several times faster.  Large inputs therefore go through the instance's device
                // input buffer (image i), enqueued on the same stream right before the first kernel group.
                if (direct_io && cur == lead && in_bytes_ >= kDmaInputBytes) {
                    check(cudaMemcpyAsync(static_cast<char*>(pb_instance_input_dev(inst_)) + (size_t)i * in_bytes_, io, in_bytes_,
                                          cudaMemcpyHostToDevice, st));
                    ins[i] = nullptr;
                }
                outs[i] = direct_io ? io + get_output_offset() : nullptr;
            }
            if (pb_instance_launch_group_batched(inst_, cur - lead, gang_n_, st, get_id(), get_finished_block_notifier(), ins, outs) != PB_OK)
                set_error(PB_ERR_CUDA);
        } else {
            if (!resident_) check(cudaMemcpyAsync(io_ptr_ + get_output_offset(), pb_instance_output_dev(inst_), out_bytes_, cudaMemcpyDeviceToHost, st));
        }
    }

    bool has_next() const override { return next_ < num_groups_ + (copy_stages_ ? 2 : 0); }

  private:
    static constexpr size_t kDmaInputBytes = 64 * 1024;
    void check(cudaError_t e) { if (e != cudaSuccess) set_error(PB_ERR_CUDA); }

    // Declares stage `next_` (resources, copy or compute, pre-notify on the last one).
    void declare() {
        const int n = num_groups_;
        const int lead = copy_stages_ ? 1 : 0;
        const int total = n + 2 * lead;
        if (next_ >= total) return;
        if (next_ < lead || next_ >= lead + n) {
            set_is_mem();
            set_gang_decls(nullptr, 1);
        } else {
            unset_is_mem();
            const llis::job::StageDecl* row = &decls_[(size_t)(next_ - lead) * cap_];
            set_next_stage(row[gang_n_ - 1]);
            set_gang_decls(row, (unsigned)cap_);
        }
        if (next_ == total - 1) set_pre_notify();
    }

    // Instances by the server that owns them: the job objects themselves are never destroyed (the plugin ABI has no
    // virtual destructor and the reference pools instances for ever, src/server/registered_job.cpp:91-93), but a
    // server that goes away gives the device memory of its instances back through pb_plugin_release().
    static std::map<void*, std::vector<pb_instance*>>& registry() {
        static std::map<void*, std::vector<pb_instance*>> r;
        return r;
    }
    static std::mutex& registry_mu() {
        static std::mutex mu;
        return mu;
    }
    static void remember(void* owner, pb_instance* inst) {
        std::lock_guard<std::mutex> lk(registry_mu());
        registry()[owner].push_back(inst);
    }

  public:
    static void release_all(void* owner) {
        std::vector<pb_instance*> mine;
        {
            std::lock_guard<std::mutex> lk(registry_mu());
            auto it = registry().find(owner);
            if (it == registry().end()) return;
            mine.swap(it->second);
            registry().erase(it);
        }
        for (pb_instance* i : mine) pb_instance_destroy(i);
    }

  private:
    static pb_model* shared_model(int device, const std::string& path) {
        static std::mutex mu;
        static std::map<std::pair<int, std::string>, pb_model*> cache;
        std::lock_guard<std::mutex> lk(mu);
        auto key = std::make_pair(device, path);
        auto it = cache.find(key);
        if (it != cache.end()) return it->second;
        pb_model* m = nullptr;
        int precision = -1;
        if (const char* p = std::getenv("PB_PRECISION")) precision = std::atoi(p);
        if (pb_model_load(path.c_str(), device, precision, &m) != PB_OK) return nullptr;
        cache[key] = m;
        return m;
    }

    std::string name_;
    size_t in_bytes_, out_bytes_;
    pb_instance* inst_ = nullptr;
    std::vector<llis::job::StageDecl> decls_;      // [group][gang size - 1]
    int num_groups_ = 0;
    int cap_ = 1;          // images the instance holds = largest gang this job can lead
    int gang_n_ = 1;       // members of the gang this job currently leads (1 = alone)
    char* io_ptr_ = nullptr;
    int next_ = 0;
    bool resident_ = false;
    bool copy_stages_ = false;
};

}  // namespace pbjobs

#define PB_DEFINE_MODEL_JOB(NAME, IN_FLOATS, OUT_FLOATS)                                             \
    extern "C" __attribute__((visibility("default"))) llis::job::Job* init_job() {                  \
        return new pbjobs::ModelJob(NAME, IN_FLOATS, OUT_FLOATS);                                    \
    }                                                                                                \
    /* optional: a server that is being destroyed hands back the device memory of its instances */  \
    extern "C" __attribute__((visibility("default"))) void pb_plugin_release(void* owner) {         \
        pbjobs::ModelJob::release_all(owner);                                                        \
    }
