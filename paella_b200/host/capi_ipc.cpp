// C ABI over the client<->server IPC pieces (shared-memory byte ring, client library), so that
// tests and tools can drive them without C++.
#include <llis/client/client.h>
#include <llis/ipc/shm_channel.h>

#include <exception>

#include "../csrc/pb_common.h"

struct pb_shm_channel { llis::ipc::ShmChannel ch; };
struct pb_client {
    llis::client::Client client;
    std::vector<llis::client::JobRef*> jobs;
    explicit pb_client(const char* name) : client(name) {}
};

#define PB_TRY(stmt)                                              \
    try { stmt; } catch (const std::exception& e) {               \
        pb::set_error("%s", e.what());                            \
        return PB_ERR_IO;                                         \
    }

extern "C" {

int pb_shm_channel_open(const char* name, size_t size, pb_shm_channel** out) {
    PB_REQUIRE(name && out, "pb_shm_channel_open: NULL argument");
    pb_shm_channel* c = new pb_shm_channel();
    try { c->ch.connect(name, size); } catch (const std::exception& e) { pb::set_error("%s", e.what()); delete c; return PB_ERR_IO; }
    *out = c;
    return PB_OK;
}
void pb_shm_channel_close(pb_shm_channel* c) { delete c; }
int pb_shm_channel_write(pb_shm_channel* c, const void* buf, size_t n, uint64_t max_spins) {
    PB_REQUIRE(c && (buf || n == 0), "pb_shm_channel_write: NULL argument");
    return c->ch.write(buf, n, max_spins) ? PB_OK : PB_ERR_TIMEOUT;
}
int pb_shm_channel_read(pb_shm_channel* c, void* buf, size_t n, uint64_t max_spins) {
    PB_REQUIRE(c && (buf || n == 0), "pb_shm_channel_read: NULL argument");
    return c->ch.read(buf, n, max_spins) ? PB_OK : PB_ERR_TIMEOUT;
}
int pb_shm_channel_can_read(pb_shm_channel* c) { return c && c->ch.can_read() ? 1 : 0; }
void pb_shm_channel_lock(pb_shm_channel* c) { if (c) c->ch.acquire_writer_lock(); }
void pb_shm_channel_unlock(pb_shm_channel* c) { if (c) c->ch.release_writer_lock(); }

int pb_client_connect(const char* server_name, pb_client** out) {
    PB_REQUIRE(server_name && out, "pb_client_connect: NULL argument");
    PB_TRY(*out = new pb_client(server_name));
    return PB_OK;
}
void pb_client_close(pb_client* c) { delete c; }
uint32_t pb_client_id(const pb_client* c) { return c ? c->client.get_client_id() : 0; }

int pb_client_register_job(pb_client* c, const char* plugin_path, uint32_t* job_out, size_t* in_bytes, size_t* out_bytes) {
    PB_REQUIRE(c && plugin_path && job_out, "pb_client_register_job: NULL argument");
    PB_TRY(c->jobs.push_back(c->client.register_job(plugin_path)));
    *job_out = (uint32_t)c->jobs.size() - 1;
    if (in_bytes) *in_bytes = c->jobs.back()->get_job()->get_input_size();
    if (out_bytes) *out_bytes = c->jobs.back()->get_job()->get_output_size();
    return PB_OK;
}

int pb_client_create_instance(pb_client* c, uint32_t job, uint64_t* instance_out, void** in_ptr, void** out_ptr) {
    PB_REQUIRE(c && job < c->jobs.size() && instance_out, "pb_client_create_instance: bad arguments");
    llis::client::JobInstanceRef* r = nullptr;
    PB_TRY(r = c->jobs[job]->create_instance());
    *instance_out = (uint64_t)(uintptr_t)r;
    if (in_ptr) *in_ptr = r->get_input_ptr();
    if (out_ptr) *out_ptr = r->get_output_ptr();
    return PB_OK;
}

int pb_client_launch(pb_client* c, uint64_t instance) {
    PB_REQUIRE(c && instance, "pb_client_launch: bad arguments");
    PB_TRY(reinterpret_cast<llis::client::JobInstanceRef*>((uintptr_t)instance)->launch());
    return PB_OK;
}

int pb_client_wait(pb_client* c, int timeout_ms, uint64_t* instance_out) {
    PB_REQUIRE(c && instance_out, "pb_client_wait: bad arguments");
    llis::client::JobInstanceRef* r = nullptr;
    PB_TRY(r = timeout_ms < 0 ? c->client.wait() : c->client.wait_timeout(timeout_ms));
    *instance_out = (uint64_t)(uintptr_t)r;
    return r ? 1 : 0;
}

int pb_client_kill_server(pb_client* c) {
    PB_REQUIRE(c != nullptr, "pb_client_kill_server: NULL client");
    PB_TRY(c->client.kill_server());
    return PB_OK;
}

int pb_client_profiler_cmd(pb_client* c, uint32_t cmd, const char* path) {
    PB_REQUIRE(c != nullptr && cmd <= (uint32_t)llis::ProfilerMsgType::SAVE, "pb_client_profiler_cmd: bad argument");
    PB_REQUIRE(cmd != (uint32_t)llis::ProfilerMsgType::SAVE || (path && path[0]), "pb_client_profiler_cmd: SAVE needs a path prefix");
    PB_TRY(c->client.profiler_cmd((llis::ProfilerMsgType)cmd, path ? path : ""));
    return PB_OK;
}

}  // extern "C"
