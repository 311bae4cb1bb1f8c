// Thread-local context slots and the host faces of the ring / notifier classes.
#include <llis/job/context.h>
#include <llis/job/finished_block_notifier.h>
#include <llis/server/scheduler.h>

#include <stdexcept>
#include <string>

#include "paella_b200.h"
#include "registry.h"

namespace llis {
namespace job {

namespace {
thread_local Job* t_current_job = nullptr;
thread_local ipc::Gpu2SchedChannel* t_channel = nullptr;
thread_local int t_device = 0;
thread_local bool t_device_resident = false;
thread_local void* t_owner = nullptr;
thread_local unsigned t_max_gang = 1;
thread_local Job* const* t_gang = nullptr;
thread_local unsigned t_gang_n = 0;
}  // namespace

Job* Context::get_current_job() { return t_current_job; }
void Context::set_current_job(Job* job) { t_current_job = job; }
ipc::Gpu2SchedChannel* Context::get_gpu2sched_channel() { return t_channel; }
void Context::set_gpu2sched_channel(ipc::Gpu2SchedChannel* ch) { t_channel = ch; }
int Context::get_device() { return t_device; }
void Context::set_device(int device) { t_device = device; }
bool Context::device_resident() { return t_device_resident; }
void Context::set_device_resident(bool v) { t_device_resident = v; }
void* Context::get_owner() { return t_owner; }
void Context::set_owner(void* owner) { t_owner = owner; }
unsigned Context::max_gang() { return t_max_gang; }
void Context::set_max_gang(unsigned n) { t_max_gang = n >= 1 ? n : 1; }
Job* const* Context::get_gang(unsigned* num_followers) {
    if (num_followers) *num_followers = t_gang_n;
    return t_gang;
}
void Context::set_gang(Job* const* followers, unsigned num_followers) {
    t_gang = num_followers ? followers : nullptr;
    t_gang_n = followers ? num_followers : 0;
}

FinishedBlockNotifier* FinishedBlockNotifier::create_array(unsigned num, ipc::Gpu2SchedChannel* channel) {
    void* dev = nullptr;
    if (pb_notifier_create_array(channel->handle(), num, &dev) != PB_OK) throw std::runtime_error(pb_last_error());
    return static_cast<FinishedBlockNotifier*>(dev);
}
void FinishedBlockNotifier::free_array(FinishedBlockNotifier* ptr) { pb_notifier_free_array(ptr); }

}  // namespace job

namespace ipc {

Gpu2SchedChannel::Gpu2SchedChannel(size_t count, int device) { connect(count, device); }
Gpu2SchedChannel::~Gpu2SchedChannel() { disconnect(); }

void Gpu2SchedChannel::connect(size_t count, int device) {
    disconnect();
    if (pb_ring_create(device, count, &ring_) != PB_OK) throw std::runtime_error(pb_last_error());
}
void Gpu2SchedChannel::disconnect() {
    if (ring_) pb_ring_destroy(ring_);
    ring_ = nullptr;
}
bool Gpu2SchedChannel::try_read(job::InstrumentInfo* out) {
    uint64_t rec;
    const int n = pb_ring_poll(ring_, &rec, 1);
    if (n < 0) throw std::runtime_error(pb_last_error());
    if (n == 0) return false;
    *out = job::InstrumentInfo::unpack(rec);
    return true;
}
bool Gpu2SchedChannel::read(job::InstrumentInfo* out, uint64_t max_spins) {
    for (uint64_t i = 0; max_spins == 0 || i < max_spins; ++i)
        if (try_read(out)) return true;
    return false;
}
Gpu2SchedChannelDev Gpu2SchedChannel::device_view() const {
    Gpu2SchedChannelDev v{};
    if (pb_ring_device_view(ring_, &v, sizeof(v)) != PB_OK) throw std::runtime_error(pb_last_error());
    return v;
}

}  // namespace ipc

namespace server {

std::unique_ptr<Scheduler> Scheduler::create(const std::string& name, const SchedulerConfig& cfg, SchedulerHost* host) {
    if (name.empty() || name == "full3") return make_scheduler_full3(cfg, host);
    if (name == "fifo") return make_scheduler_fifo(cfg, host);
    if (name == "fifo2") return make_scheduler_fifo2(cfg, host);
    return nullptr;
}

}  // namespace server
}  // namespace llis
