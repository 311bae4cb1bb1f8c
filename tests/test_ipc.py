"""Client<->server IPC on CPU: the shared-memory byte ring against the reference's own fixtures
(ints 0..9999 in order through a 64-byte ring, same process and two processes:
tests/ipc/shm_channel/shmc_read_write_same_proc.cpp:5-31, shmc_read.cpp + shmc_write.cpp), and the
client library's wire messages against a server played by the test."""
import ctypes as C
import multiprocessing as mp
import os
import socket
import struct
import threading

import pytest

from paella_b200 import capi

SPINS = 1 << 28


def _open(name, size=0):
    L = capi.load()
    h = C.c_void_p()
    capi.check(L.pb_shm_channel_open(name.encode(), size, C.byref(h)), "pb_shm_channel_open")
    return h


def _write(h, data: bytes):
    capi.check(capi.load().pb_shm_channel_write(h, data, len(data), SPINS), "write")


def _read(h, n) -> bytes:
    buf = C.create_string_buffer(n)
    capi.check(capi.load().pb_shm_channel_read(h, buf, n, SPINS), "read")
    return buf.raw


def _uniq(tag):
    return f"pbtest-{tag}-{os.getpid()}"


def test_ints_in_order_through_a_64_byte_ring_two_threads():
    name = _uniq("thr")
    r = _open(name, 64)
    w = _open(name)
    got = []

    def reader():
        for _ in range(10000):
            got.append(struct.unpack("<i", _read(r, 4))[0])

    t = threading.Thread(target=reader)
    t.start()
    for i in range(10000):
        _write(w, struct.pack("<i", i))
    t.join(60)
    assert got == list(range(10000))
    capi.load().pb_shm_channel_close(w)
    capi.load().pb_shm_channel_close(r)


def _writer_proc(name, lo, hi, tag, locked):
    L = capi.load()
    w = _open(name)
    for i in range(lo, hi):
        rec = struct.pack("<ii", tag, i) * 3          # 24 bytes: must never interleave with the other writer
        if locked:
            L.pb_shm_channel_lock(w)
        _write(w, rec)
        if locked:
            L.pb_shm_channel_unlock(w)
    L.pb_shm_channel_close(w)


def test_two_processes_and_records_larger_than_the_ring():
    name = _uniq("proc")
    r = _open(name, 64)
    p = mp.get_context("fork").Process(target=_writer_proc, args=(name, 0, 3000, 7, False))
    p.start()
    for i in range(3000):
        assert struct.unpack("<6i", _read(r, 24)) == (7, i) * 3
    p.join(60)
    assert p.exitcode == 0
    # one message larger than the ring: the copy proceeds in pieces while the reader drains
    big = bytes(range(256)) * 4
    t = threading.Thread(target=lambda: _write(_open(name), big))
    t.start()
    assert _read(r, len(big)) == big
    t.join(30)
    assert capi.load().pb_shm_channel_can_read(r) == 0
    capi.load().pb_shm_channel_close(r)


def test_writer_lock_keeps_two_writers_records_whole():
    name = _uniq("lock")
    r = _open(name, 256)
    ctx = mp.get_context("fork")
    ps = [ctx.Process(target=_writer_proc, args=(name, 0, 2000, tag, True)) for tag in (1, 2)]
    for p in ps:
        p.start()
    nxt = {1: 0, 2: 0}
    for _ in range(4000):
        rec = struct.unpack("<6i", _read(r, 24))
        tag, i = rec[0], rec[1]
        assert rec == (tag, i) * 3 and i == nxt[tag]
        nxt[tag] += 1
    for p in ps:
        p.join(60)
    assert nxt == {1: 2000, 2: 2000}
    capi.load().pb_shm_channel_close(r)


def test_bounded_read_times_out_instead_of_hanging():
    name = _uniq("to")
    r = _open(name, 32)
    buf = C.create_string_buffer(4)
    assert capi.load().pb_shm_channel_read(r, buf, 4, 1000) == -5
    capi.load().pb_shm_channel_close(r)


def test_client_library_wire_messages_against_a_played_server():
    """REGISTER_CLIENT / REGISTER_JOB / GROW_POOL / LAUNCH_JOB as the reference's client sends them
    (src/client/client.cpp:44-51, job_ref.cpp:31-41,70-101, job_instance_ref.cpp:31-45) and the two
    completion signals (server.cpp:158-167)."""
    L = capi.load()
    server = _uniq("srv")
    c2s = _open("c2s:" + server, 1024)
    client = C.c_void_p()
    res = {}
    t = threading.Thread(target=lambda: res.setdefault("rc", L.pb_client_connect(server.encode(), C.byref(client))))
    t.start()
    # --- REGISTER_CLIENT {u32 msg = 0, u32 temporary id}
    msg, tmp_id = struct.unpack("<II", _read(c2s, 8))
    assert msg == 0
    tmp = _open(f"s2c:{server}:{tmp_id}")                     # the client's temporary 8-byte ring
    s2c = _open(f"s2c:{server}:0", 4096)                      # permanent ring for client id 0
    _write(tmp, struct.pack("<I", 0))
    t.join(30)
    assert res["rc"] == 0 and L.pb_client_id(client) == 0
    # --- REGISTER_JOB {u32 1, u32 client id, string path, string shm name} -> job_ref_id on s2c
    plugin = capi.plugin_path("tvm_mnist")
    job, ib, ob = C.c_uint32(99), C.c_size_t(), C.c_size_t()
    t = threading.Thread(target=lambda: res.setdefault("rj", L.pb_client_register_job(client, plugin.encode(), C.byref(job), C.byref(ib), C.byref(ob))))
    t.start()
    msg, cid = struct.unpack("<II", _read(c2s, 8))
    assert (msg, cid) == (1, 0)
    n = struct.unpack("<Q", _read(c2s, 8))[0]
    assert _read(c2s, n).decode() == plugin
    n = struct.unpack("<Q", _read(c2s, 8))[0]
    shm_name = _read(c2s, n).decode()
    assert shm_name.startswith("llis:shm:0:")
    _write(s2c, struct.pack("<I", 5))                         # job_ref_id 5
    # --- GROW_POOL {u32 3, u32 job_ref_id, size_t bytes}: fixed 30 638 080-byte chunk
    msg, jid, nbytes = struct.unpack("<IIQ", _read(c2s, 16))
    assert (msg, jid, nbytes) == (3, 5, 30638080)
    t.join(30)
    assert res["rj"] == 0 and (ib.value, ob.value) == (3136, 40)
    assert os.path.getsize("/dev/shm/" + shm_name) == 30638080
    # --- LAUNCH_JOB {u32 2, u32 job_ref_id, int chunk, size_t offset, pointer}
    inst, pin, pout = C.c_uint64(), C.c_void_p(), C.c_void_p()
    capi.check(L.pb_client_create_instance(client, job, C.byref(inst), C.byref(pin), C.byref(pout)), "create_instance")
    assert pout.value - pin.value == 3136
    capi.check(L.pb_client_launch(client, inst), "launch")
    msg, jid, chunk, off, ptr = struct.unpack("<IIiQQ", _read(c2s, 28))
    assert (msg, jid, chunk) == (2, 5, 0) and off % 3176 == 0 and ptr == inst.value
    # --- completion: datagram (job started) then the pointer on s2c (job ended)
    got = C.c_uint64()
    assert L.pb_client_wait(client, 50, C.byref(got)) == 0                     # nothing yet
    sk = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
    sk.sendto(b"\x01", b"\0" + f"llis-socket-s2c-{server}-0".encode().ljust(107, b"\0"))
    _write(s2c, struct.pack("<Q", ptr))
    assert L.pb_client_wait(client, 2000, C.byref(got)) == 1 and got.value == inst.value
    # --- a late wake-up: entries already in the ring are handed out at once; the datagrams they owe are
    #     swallowed when they arrive, and the next datagram pairs with the next entry again
    addr = b"\0" + f"llis-socket-s2c-{server}-0".encode().ljust(107, b"\0")
    _write(s2c, struct.pack("<Q", 0x1111))
    _write(s2c, struct.pack("<Q", 0x2222))
    assert L.pb_client_wait(client, 0, C.byref(got)) == 1 and got.value == 0x1111
    assert L.pb_client_wait(client, 0, C.byref(got)) == 1 and got.value == 0x2222
    sk.sendto(b"\x01", addr)
    sk.sendto(b"\x01", addr)                                  # the two owed datagrams
    assert L.pb_client_wait(client, 50, C.byref(got)) == 0      # both swallowed, nothing to hand out
    sk.sendto(b"\x01", addr)                                  # pre-notification of a third job ...
    threading.Timer(0.2, lambda: _write(s2c, struct.pack("<Q", 0x3333))).start()   # ... whose entry follows
    assert L.pb_client_wait(client, 2000, C.byref(got)) == 1 and got.value == 0x3333
    assert L.pb_client_wait(client, 50, C.byref(got)) == 0
    # --- EXIT_CMD {u32 7}
    capi.check(L.pb_client_kill_server(client), "kill_server")
    assert struct.unpack("<I", _read(c2s, 4))[0] == 7
    L.pb_client_close(client)
    for h in (tmp, s2c, c2s):
        L.pb_shm_channel_close(h)
    os.unlink("/dev/shm/" + shm_name)
