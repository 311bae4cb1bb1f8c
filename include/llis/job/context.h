// Per-server-thread context a plugin can query while the server calls into it.
//
// Same role and accessor names as the reference's include/llis/job/context.h:10-53
// (process-global statics there).  Here the slots are thread-local: one server
// (scheduler + pools) runs per GPU, each on its own thread of one process, and every
// plugin call happens on the thread of the server that owns the job.
#pragma once

#include <llis/ipc/shm_primitive_channel.h>
#include <llis/job/job.h>

namespace llis {
namespace job {

class Context {
  public:
    static Job* get_current_job();
    static void set_current_job(Job* job);
    static ipc::Gpu2SchedChannel* get_gpu2sched_channel();
    static void set_gpu2sched_channel(ipc::Gpu2SchedChannel* ch);
    // CUDA device of the calling server thread (the reference hard-wires device 0).
    static int get_device();
    static void set_device(int device);
    // True when requests' inputs are already resident in device memory and results stay
    // there: model jobs then skip their host<->device copies (benchmark mode).
    static bool device_resident();
    static void set_device_resident(bool v);
    // Gangs.  max_gang: how many jobs of one type the server's scheduler may run as one launch per stage
    // (1 = never; a plugin sizes its buffers for it at full_init).  get_gang: during run_next() of a gang's
    // leader, the other members (same type, same stage, their io_ptr given at init()); NULL / 0 otherwise.
    // The server on whose behalf the plugin is being called (an opaque token; NULL outside a server).  A plugin that
    // exports `extern "C" void pb_plugin_release(void* owner)` is called with it when that server is destroyed and
    // may free what its jobs of that server hold on the device.
    static void* get_owner();
    static void set_owner(void* owner);
    static unsigned max_gang();
    static void set_max_gang(unsigned n);
    static Job* const* get_gang(unsigned* num_followers);
    static void set_gang(Job* const* followers, unsigned num_followers);
};

}  // namespace job
}  // namespace llis
