// Model packs and instances: the graph executor behind the model job adapters.
//
// A pack (written by paella_b200/packer.py) is a flat operator table plus fp32 weights
// in boundary layouts (NCHW / OIHW).  Loading a pack turns it into a list of STAGES, one
// kernel launch each, with weights repacked for the kernel chosen per layer:
//   tcgen05 implicit GEMM for dense convolutions in bf16, the vectorised depthwise / pool /
//   dense / add / softmax kernels, direct convolution as the fp32 path.
// An instance owns the activation buffers of one in-flight request.
// Stages are handed to the scheduler in GROUPS; a group is replayed as one CUDA graph whose kernels
// form a chain ordered by dependence depth, independent tensor-core convolutions sharing a launch.
//
// Replaces what the reference gets from tvm::runtime (Module::LoadFromFile, "run",
// "get_input", "get_output": jobs/tvm_mnist/tvm_mnist.cpp:24-33); one stage here is one of
// the kernels its graph executor launches between two scheduler yields.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "launch_slot.cuh"
#include "ops.h"
#include "pb_common.h"

namespace {

constexpr uint32_t kNone = 0xFFFFFFFFu;
enum { OP_CONV = 1, OP_DENSE = 2, OP_MAXPOOL = 3, OP_AVGPOOL = 4, OP_GAP = 5, OP_ADD = 6, OP_SOFTMAX = 7, OP_AFFINE = 8, OP_DETECT = 9 };

struct PackOp {
    uint32_t type, in0, in1, out, rsv0, out_c_off, cin, cout, r, s, stride_h, stride_w, pad_h, pad_w, groups, act, flags,
        rsv1, w_off_lo, w_off_hi, b_off_lo, b_off_hi, dil_h, dil_w;     // dilation 0 reads as 1
};
static_assert(sizeof(PackOp) == 96, "pack op record is 96 bytes");

struct TensorInfo {
    int C, H, W, Cs;
    size_t offset;   // in the activation arena (bytes); unused for the fp32 output tensor
    size_t bytes;
};

struct Stage {
    int kind;
    pb_op_params p;           // pointers hold arena OFFSETS (+1) until an instance resolves them
    size_t x_off, y_off, res_off;
    bool x_is_input, y_is_output, has_res;
    void* w_dev = nullptr;
    float* bias_dev = nullptr;
    pb::ConvUmmaPlan* plan = nullptr;
    pb_launch_info info;
    std::string name;
    int out_tensor;
    int in_tensor = -1, res_tensor = -1;   // tensors read (-1: the request input / none)
    size_t scratch_off = 0;                // this stage's private slice of the instance's scratch buffer
};

}  // namespace

struct pb_model {
    int device = 0;
    int dtype = 1;
    std::string name;
    std::vector<TensorInfo> tensors;
    std::vector<Stage> stages;
    int t_in = 0, t_out = 0;
    size_t arena_bytes = 0;
    size_t scratch_bytes = 0;     // sum of the stages' scratch requirements: every split-K layer has its own
                                  // slice, so kernels of parallel branches never share partial tiles
    size_t in_floats = 0, out_floats = 0;
    bool mnist_fused = false;
    // Stage groups: what the job adapter hands to the scheduler as ONE stage.  A group of several
    // kernels is replayed as a CUDA graph (one driver call); only its last kernel notifies.
    // `launches`: the group's kernels in launch order (by dependence depth); an entry with several
    // stages is ONE grouped launch of independent tensor-core convolutions.
    struct Group { int first, count; pb_launch_info info; std::vector<std::vector<int>> launches; };
    std::vector<Group> groups;
    bool fuse_branches = false;
    bool persist = false;       // tensor-core launches of the stage graphs run the persistent (multi-tile) kernel
    // fused MNIST weights (device)
    float *w1 = nullptr, *b1 = nullptr, *w2 = nullptr, *b2 = nullptr, *wd = nullptr, *bd = nullptr;
    std::vector<void*> allocs;
};

// Everything of an instance that depends on how many images one launch carries.  An instance of
// capacity `cap` can run any batch nb <= cap (a gang of nb requests of the model as ONE set of launches:
// the tensor-core convolutions see nb * pixels rows, the other kernels put the image on blockIdx.y);
// it has one variant per batch size it has been asked for.
struct Variant {
    int nb = 1;
    std::vector<pb_op_params> params;       // per stage, pointers resolved
    std::vector<pb::ConvUmmaXMap*> xmaps;   // per stage: im2col descriptor of the stage's input (tensor-core convs)
    std::vector<pb_launch_info> group_info; // per group, for this batch
    std::vector<cudaGraphExec_t> graphs;    // per group; NULL = single kernel, launched directly
    std::vector<std::vector<pb::ConvUmmaMulti*>> multis;   // [group][launch]: descriptor table of a grouped conv launch
    char* scratch = nullptr;                // split-K scratch, one private slice per stage that splits at this batch
};

struct pb_instance {
    pb_model* m = nullptr;
    int cap = 1;                            // images the buffers hold
    char* arena = nullptr;                  // tensor t: cap images back to back at cap * offset(t)
    float* in_dev = nullptr;                // [cap][input floats]
    float* out_dev = nullptr;               // [cap][output floats]
    pb::LaunchSlot* slot_host = nullptr;    // pinned mirror, filled before each graph launch
    pb::LaunchSlot* slot_dev = nullptr;
    std::vector<Variant*> variants;         // [nb - 1], NULL until built
};

namespace {

int upload(pb_model* m, const void* host, size_t bytes, void** dev_out) {
    void* d = nullptr;
    PB_CUDA(cudaMalloc(&d, bytes > 0 ? bytes : 16));
    m->allocs.push_back(d);
    if (bytes > 0) PB_CUDA(cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice));
    *dev_out = d;
    return PB_OK;
}

bool env_flag(const char* name, bool dflt) {
    const char* v = getenv(name);
    if (!v || !*v) return dflt;
    return !(v[0] == '0' || v[0] == 'n' || v[0] == 'N' || v[0] == 'f' || v[0] == 'F');
}

bool is_mnist_topology(const std::vector<PackOp>& ops, const std::vector<TensorInfo>& t, int t_in) {
    if (ops.size() != 5) return false;
    const PackOp& c1 = ops[0]; const PackOp& p1 = ops[1]; const PackOp& c2 = ops[2]; const PackOp& p2 = ops[3]; const PackOp& fc = ops[4];
    if (t[t_in].C != 1 || t[t_in].H != 28 || t[t_in].W != 28) return false;
    auto conv5 = [](const PackOp& o, uint32_t ci, uint32_t co) {
        return o.type == OP_CONV && o.cin == ci && o.cout == co && o.r == 5 && o.s == 5 && o.stride_h == 1 && o.stride_w == 1 &&
               o.pad_h == 2 && o.pad_w == 2 && o.groups == 1 && o.act == 1 && o.in1 == kNone && o.out_c_off == 0;
    };
    auto pool = [](const PackOp& o, uint32_t k) {
        return o.type == OP_MAXPOOL && o.r == k && o.s == k && o.stride_h == k && o.stride_w == k && o.pad_h == 0 && o.pad_w == 0 &&
               o.out_c_off == 0;
    };
    return conv5(c1, 1, 8) && pool(p1, 2) && conv5(c2, 8, 16) && pool(p2, 3) && fc.type == OP_DENSE && fc.cin == 256 &&
           fc.cout == 10 && fc.act == 0;
}


// Launches that go through a descriptor table (ConvUmmaMulti): several tensor-core convolutions in one grid,
// and with the persistent kernel every tensor-core convolution of a stage graph.
bool uses_multi(const pb_model* m, const std::vector<int>& l) {
    if (l.size() > 1) return true;
    return m->persist && m->stages[(size_t)l[0]].kind == PB_STAGE_CONV_UMMA;
}

// What group `g` declares to the scheduler, from its stages' launch geometry `infos` (per stage): only the
// LAST launch of a group reports block start/end, so the declared block count is that launch's grid; the
// per-block resources are scaled so that blocks x per-block equals the largest footprint any launch of
// the group has on the GPU.
pb_launch_info group_footprint(const pb_model* m, int g, const std::vector<pb_launch_info>& infos) {
    const pb_model::Group& grp = m->groups[(size_t)g];
    pb_launch_info out;
    memset(&out, 0, sizeof(out));
    uint64_t thr = 0, smem = 0, regs = 0, tmem = 0, nb = 0;
    for (const std::vector<int>& l : grp.launches) {
        uint64_t lt = 0, ls = 0, lr = 0, lm = 0, lb = 0;
        uint32_t max_tmem = 0;
        for (int i : l) {
            const pb_launch_info& li = infos[(size_t)i];
            lb += li.num_blocks;
            lt += (uint64_t)li.num_blocks * li.threads_per_block;
            ls += (uint64_t)li.num_blocks * li.smem_per_block;
            lr += (uint64_t)li.num_blocks * li.threads_per_block * li.regs_per_thread;
            lm += (uint64_t)li.num_blocks * li.tmem_cols_per_block;
            max_tmem = std::max(max_tmem, li.tmem_cols_per_block);
            out.flops += li.flops;
            out.bytes += li.bytes;
        }
        if (uses_multi(m, l)) {
            // the launch's tiles (lb) are walked by fewer, longer-lived CTAs
            pb_launch_info pf;
            pb::conv_umma_persist_footprint((uint32_t)lb, max_tmem, &pf);
            if (m->persist && 2u * max_tmem <= 512u) {
                lb = pf.num_blocks;
                lt = lb * pf.threads_per_block;
                ls = lb * pf.smem_per_block;
                lr = lt * pf.regs_per_thread;
                lm = lb * pf.tmem_cols_per_block;
            }
        }
        thr = std::max(thr, lt); smem = std::max(smem, ls); regs = std::max(regs, lr); tmem = std::max(tmem, lm);
        nb = lb;
    }
    out.kind = grp.count == 1 ? infos[(size_t)grp.first].kind : 0xFFFFu;
    out.num_blocks = (uint32_t)nb;
    out.threads_per_block = (uint32_t)pb::ceil_div<uint64_t>(thr, nb);
    out.smem_per_block = (uint32_t)pb::ceil_div<uint64_t>(smem, nb);
    out.regs_per_thread = (uint32_t)pb::ceil_div<uint64_t>(regs, (uint64_t)out.threads_per_block * nb);
    out.tmem_cols_per_block = (uint32_t)pb::ceil_div<uint64_t>(tmem, nb);
    return out;
}

// Splits the stage list into groups of at most PB_STAGE_GROUP kernels (default 48; 1 = one kernel per
// scheduler stage, the reference's granularity) and derives each group's stage declaration.
void build_groups(pb_model* m) {
    int gs = 48;      // measured on the headline mix: 24 -> 221k req/s with the host thread 94 % busy, 48 -> 225k at 79 %
    if (const char* e = getenv("PB_STAGE_GROUP")) gs = atoi(e);
    if (gs < 1) gs = 1;
    // Independent tensor-core convolutions of equal dependence depth share one launch, unless the
    // graphs are captured with parallel branches (PB_GRAPH_BRANCHES=1) or PB_FUSE_BRANCHES=0.
    m->fuse_branches = env_flag("PB_FUSE_BRANCHES", true) && !env_flag("PB_GRAPH_BRANCHES", false) && pb::conv_umma_multi_available();
    m->persist = !env_flag("PB_GRAPH_BRANCHES", false) && pb::conv_umma_multi_available() && pb::conv_umma_persist_enabled();
    const int n = (int)m->stages.size();
    std::vector<std::vector<int>> writers(m->tensors.size());
    for (int first = 0; first < n; first += gs) {
        pb_model::Group g;
        g.first = first;
        g.count = first + gs <= n ? gs : n - first;
        memset(&g.info, 0, sizeof(g.info));
        // dependence depth inside the group
        std::vector<int> level((size_t)g.count, 0);
        for (auto& w : writers) w.clear();
        for (int i = first; i < first + g.count; ++i) {
            const Stage& st = m->stages[i];
            int lv = 0;
            for (int t : {st.in_tensor, st.res_tensor})
                if (t >= 0)
                    for (int w : writers[(size_t)t]) lv = std::max(lv, level[(size_t)(w - first)] + 1);
            level[(size_t)(i - first)] = lv;
            writers[(size_t)st.out_tensor].push_back(i);
        }
        std::vector<int> order((size_t)g.count);
        for (int i = 0; i < g.count; ++i) order[(size_t)i] = first + i;
        if (m->fuse_branches)
            std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return level[(size_t)(a - first)] < level[(size_t)(b - first)]; });
        // PB_FUSE_POOLS=1 (off by default; not with the persistent kernel): a 3x3 pooling layer joins the grouped launch of
        // the convolutions of its depth.  A launch that contains a pooling layer always starts with a convolution.
        // Measured: same bits, a lone Inception-v3 request 885 -> 870 us, but 26.9k -> 17.4k req/s with 96 requests in
        // flight: a pooling block then holds a whole convolution slot of its SM (the launch's 73 KB of shared memory) while
        // it waits on loads, and there are 600-900 of them per launch at 8 images.
        const bool fuse_pools = m->fuse_branches && !m->persist && env_flag("PB_FUSE_POOLS", false);
        for (int s : order) {
            const Stage& st = m->stages[s];
            const bool conv_ok = st.kind == PB_STAGE_CONV_UMMA && !st.x_is_input && !st.y_is_output;
            const bool pool_ok = fuse_pools && !st.x_is_input && !st.y_is_output && pb::conv_umma_pool_fusable(st.kind, &st.p);
            const bool fusable = m->fuse_branches && (conv_ok || pool_ok);
            if (fusable && !g.launches.empty()) {
                std::vector<int>& prev = g.launches.back();
                const Stage& ps = m->stages[prev.front()];
                const bool prev_fusable = ps.kind == PB_STAGE_CONV_UMMA && !ps.x_is_input && !ps.y_is_output;
                if (prev_fusable && level[(size_t)(prev.front() - first)] == level[(size_t)(s - first)] && (int)prev.size() < 8) {
                    prev.push_back(s);
                    continue;
                }
            }
            g.launches.push_back(std::vector<int>{s});
        }
        // only the last launch of a group notifies, with the block count the group declares: it stays as the stages'
        // own launch geometry says, so a pooling layer that ended up there gets its own launch again
        if (!g.launches.empty()) {
            std::vector<int>& last = g.launches.back();
            std::vector<int> out_again;
            for (size_t k = last.size(); k-- > 1;)
                if (m->stages[last[k]].kind != PB_STAGE_CONV_UMMA) { out_again.push_back(last[k]); last.erase(last.begin() + (long)k); }
            for (size_t k = out_again.size(); k-- > 0;) g.launches.push_back(std::vector<int>{out_again[k]});
        }
        m->groups.push_back(g);
    }
    for (size_t gi = 0; gi < m->groups.size(); ++gi) {
        std::vector<pb_launch_info> infos(m->stages.size());
        for (size_t i = 0; i < m->stages.size(); ++i) infos[i] = m->stages[i].info;
        m->groups[gi].info = group_footprint(m, (int)gi, infos);
    }
}

// Launch geometry of stage `stage` when one launch carries `nb` images (scratch offered without limit).
int stage_info_batched(const pb_model* m, int stage, int nb, pb_launch_info* out) {
    const Stage& st = m->stages[(size_t)stage];
    if (st.kind == PB_STAGE_MNIST_FUSED) {
        const int rc = pb::mnist_fused_info(out);
        out->num_blocks *= (uint32_t)nb; out->flops *= (uint64_t)nb; out->bytes *= (uint64_t)nb;
        return rc;
    }
    pb_op_params p = st.p;
    p.batch = nb;
    p.scratch = (void*)16;
    p.scratch_bytes = ~0ull;
    return pb_op_info(st.kind, &p, out);
}

int launch_stage_with(pb_instance* in, const Variant& v, int stage, const pb_op_params* p, cudaStream_t stream, uint32_t job_id, void* notifier,
                      const float* mnist_x, float* mnist_y, bool pdl = false) {
    const Stage& st = in->m->stages[stage];
    switch (st.kind) {
        case PB_STAGE_MNIST_FUSED: {
            const pb_model* m = in->m;
            return pb::mnist_fused_launch(mnist_x, m->w1, m->b1, m->w2, m->b2, m->wd, m->bd, mnist_y, v.nb, stream, job_id, notifier);
        }
        case PB_STAGE_CONV_UMMA:
            return pb::conv_umma_launch_planned(st.plan, v.xmaps[stage], p, stream, job_id, notifier, nullptr, pdl);
        default:
            return pb::simple_op_launch(st.kind, p, stream, job_id, notifier, pdl);
    }
}

// A single small kernel reads the launch slot straight from the pinned host mirror (one PCIe read,
// no copy node: about 1 us less host time per launch); larger groups get a device copy first.
bool reads_host_slot(const pb_model* m, const pb_model::Group& grp, const Variant& v) {
    const unsigned blocks = m->stages[grp.first].info.num_blocks;
    return grp.count == 1 && blocks <= 4 && blocks * (unsigned)v.nb <= 16;
}

// Captures group `g` as ONE chain of launches in the group's planned order (dependence depth, then
// program order): [slot copy] -> launch 0 -> launch 1 -> ...  A launch is either one kernel or a grouped
// launch of independent tensor-core convolutions.  Every kernel after the first is a programmatic
// dependent of its predecessor: it waits (griddepcontrol.wait) for the completion of the kernel right
// before it, which itself waited for its own predecessor, so the chain order is a total order.
// The last launch is the one that notifies.
int capture_group_chain(pb_instance* in, Variant& v, int g, cudaStream_t origin, bool pdl_allowed) {
    const pb_model* m = in->m;
    const pb_model::Group& grp = m->groups[g];
    const bool host_slot = reads_host_slot(m, grp, v);
    void* const slot_ptr = host_slot ? (void*)in->slot_host : (void*)in->slot_dev;
    PB_CUDA(cudaStreamBeginCapture(origin, cudaStreamCaptureModeRelaxed));
    cudaError_t e = host_slot ? cudaSuccess
                              : cudaMemcpyAsync(in->slot_dev, in->slot_host, sizeof(pb::LaunchSlot), cudaMemcpyHostToDevice, origin);
    int rc = PB_OK;
    bool after_kernel = false;
    for (size_t li = 0; e == cudaSuccess && rc == PB_OK && li < grp.launches.size(); ++li) {
        const std::vector<int>& l = grp.launches[li];
        const bool is_last = li + 1 == grp.launches.size();
        if (v.multis[(size_t)g][li]) {
            rc = pb::conv_umma_multi_launch(v.multis[(size_t)g][li], origin, is_last ? pb::kSlotNotify : 0u, is_last ? slot_ptr : nullptr,
                                            pdl_allowed && after_kernel);
        } else {
            const int s = l[0];
            const Stage& st = m->stages[s];
            pb_op_params p = v.params[s];
            const bool reads_input = s == 0;                       // the request's input buffer
            const bool writes_output = st.y_is_output;             // the request's output buffer
            if (reads_input) p.x = nullptr;                        // NULL = take it from the launch slot
            if (writes_output) p.y = nullptr;
            uint32_t jid = 0;
            void* nfp = nullptr;
            if (is_last) { jid = pb::kSlotNotify; nfp = slot_ptr; }
            else if (reads_input || writes_output) { jid = pb::kSlotQuiet; nfp = slot_ptr; }
            const bool pdl = pdl_allowed && after_kernel && st.kind != PB_STAGE_MNIST_FUSED;
            rc = launch_stage_with(in, v, s, &p, origin, jid, nfp, nullptr, nullptr, pdl);
        }
        after_kernel = true;
    }
    cudaGraph_t graph = nullptr;
    const cudaError_t e2 = cudaStreamEndCapture(origin, &graph);
    if (rc != PB_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) { if (graph) cudaGraphDestroy(graph); return pb::cuda_fail(e, "graph capture", __FILE__, __LINE__); }
    if (e2 != cudaSuccess) return pb::cuda_fail(e2, "cudaStreamEndCapture", __FILE__, __LINE__);
    cudaGraphExec_t exec = nullptr;
    const cudaError_t e3 = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e3 != cudaSuccess) return pb::cuda_fail(e3, "cudaGraphInstantiate", __FILE__, __LINE__);
    v.graphs[g] = exec;
    return PB_OK;
}

// Captures group `g` of the instance into an executable graph.  The kernels are not chained in
// program order but by data dependence: the branches of an Inception block (or a down-sampling
// shortcut) sit on parallel paths of the graph and may run concurrently.
//   [slot copy] -> roots ...  each kernel after the producers of the tensors it reads ... -> last kernel
// The last kernel of the group (the one that notifies) is ordered after every other kernel.
// Kernels whose only dependence is the previous kernel on their path are programmatic dependents.
int capture_group(pb_instance* in, Variant& v, int g, cudaStream_t origin, bool pdl_allowed, bool parallel) {
    const pb_model* m = in->m;
    const pb_model::Group& grp = m->groups[g];
    const int first = grp.first, last = grp.first + grp.count - 1;
    constexpr int kMaxLanes = 6;
    std::vector<cudaStream_t> lanes{origin};
    std::vector<cudaEvent_t> events;
    auto new_event = [&]() { cudaEvent_t e = nullptr; cudaEventCreateWithFlags(&e, cudaEventDisableTiming); events.push_back(e); return e; };
    struct Done { int lane; cudaEvent_t ev; };
    std::vector<Done> done(grp.count, Done{-1, nullptr});          // per stage of the group
    std::vector<int> lane_tail{-1};                                // last stage launched on each lane (-1: none yet)
    std::vector<std::vector<int>> writers(m->tensors.size());      // in-group stages that wrote each tensor

    const bool host_slot = reads_host_slot(m, grp, v);
    void* const slot_ptr = host_slot ? (void*)in->slot_host : (void*)in->slot_dev;
    PB_CUDA(cudaStreamBeginCapture(origin, cudaStreamCaptureModeRelaxed));
    cudaError_t e = host_slot ? cudaSuccess
                              : cudaMemcpyAsync(in->slot_dev, in->slot_host, sizeof(pb::LaunchSlot), cudaMemcpyHostToDevice, origin);
    cudaEvent_t root = new_event();
    if (e == cudaSuccess) e = cudaEventRecord(root, origin);
    int rc = PB_OK;
    for (int s = first; e == cudaSuccess && rc == PB_OK && s <= last; ++s) {
        const Stage& st = m->stages[s];
        // in-group producers of what this stage reads
        std::vector<int> deps;
        for (int t : {st.in_tensor, st.res_tensor})
            if (t >= 0)
                for (int w : writers[t]) deps.push_back(w);
        if (s == last)                                            // the notifying kernel closes the group
            for (int w = first; w < last; ++w) deps.push_back(w);
        std::sort(deps.begin(), deps.end());
        deps.erase(std::unique(deps.begin(), deps.end()), deps.end());
        // lane: continue the path of a producer that is still its lane's tail, else a fresh lane
        int lane = -1;
        if (!parallel || s == last) lane = 0;
        for (size_t i = 0; lane < 0 && i < deps.size(); ++i) {
            const int dl = done[deps[i] - first].lane;
            if (lane_tail[dl] == deps[i]) lane = dl;
        }
        if (lane < 0) {
            for (size_t l = 0; l < lanes.size() && lane < 0; ++l)
                if (lane_tail[l] < 0 && (l > 0 || deps.empty())) lane = (int)l;
            if (lane < 0 && (int)lanes.size() < kMaxLanes) {
                cudaStream_t ns = nullptr;
                e = cudaStreamCreateWithFlags(&ns, cudaStreamNonBlocking);
                if (e != cudaSuccess) break;
                lanes.push_back(ns);
                lane_tail.push_back(-1);
                lane = (int)lanes.size() - 1;
            }
            if (lane < 0) lane = 0;
        }
        // order this lane after everything the stage depends on
        // A programmatic dependent waits (griddepcontrol.wait) for the completion of the kernel right
        // before it on its lane, which itself waited for its own predecessor: on a single lane that
        // covers every earlier kernel of the graph; with parallel lanes only a sole same-lane producer.
        bool chained = lane_tail[lane] >= 0 && (!parallel || (deps.size() == 1 && deps[0] == lane_tail[lane]));
        if (lane != 0 && lane_tail[lane] < 0 && e == cudaSuccess) e = cudaStreamWaitEvent(lanes[lane], root, 0);   // joins the capture
        for (size_t i = 0; e == cudaSuccess && i < deps.size(); ++i) {
            const Done& d = done[deps[i] - first];
            if (d.lane != lane || lane_tail[lane] != deps[i]) {
                if (d.lane != lane) e = cudaStreamWaitEvent(lanes[lane], d.ev, 0);
                chained = chained && d.lane == lane;
            }
        }
        if (e != cudaSuccess) break;

        pb_op_params p = v.params[s];
        const bool reads_input = s == 0;                       // the request's input buffer
        const bool writes_output = st.y_is_output;             // the request's output buffer
        if (reads_input) p.x = nullptr;                        // NULL = take it from the launch slot
        if (writes_output) p.y = nullptr;
        uint32_t jid = 0;
        void* nfp = nullptr;
        if (s == last) { jid = pb::kSlotNotify; nfp = slot_ptr; }
        else if (reads_input || writes_output) { jid = pb::kSlotQuiet; nfp = slot_ptr; }
        const bool pdl = pdl_allowed && chained && st.kind != PB_STAGE_MNIST_FUSED;
        rc = launch_stage_with(in, v, s, &p, lanes[lane], jid, nfp, nullptr, nullptr, pdl);
        if (rc != PB_OK) break;
        cudaEvent_t ev = new_event();
        e = cudaEventRecord(ev, lanes[lane]);
        done[s - first] = Done{lane, ev};
        lane_tail[lane] = s;
        writers[st.out_tensor].push_back(s);
    }
    cudaGraph_t graph = nullptr;
    const cudaError_t e2 = cudaStreamEndCapture(origin, &graph);
    for (cudaEvent_t ev : events) cudaEventDestroy(ev);
    for (size_t l = 1; l < lanes.size(); ++l) cudaStreamDestroy(lanes[l]);
    if (rc != PB_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) { if (graph) cudaGraphDestroy(graph); return pb::cuda_fail(e, "graph capture", __FILE__, __LINE__); }
    if (e2 != cudaSuccess) return pb::cuda_fail(e2, "cudaStreamEndCapture", __FILE__, __LINE__);
    cudaGraphExec_t exec = nullptr;
    const cudaError_t e3 = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e3 != cudaSuccess) return pb::cuda_fail(e3, "cudaGraphInstantiate", __FILE__, __LINE__);
    v.graphs[g] = exec;
    return PB_OK;
}

void destroy_variant(Variant* v) {
    if (!v) return;
    for (pb::ConvUmmaXMap* x : v->xmaps) pb::conv_umma_xmap_destroy(x);
    for (cudaGraphExec_t g : v->graphs) if (g) cudaGraphExecDestroy(g);
    for (auto& l : v->multis) for (pb::ConvUmmaMulti* mu : l) pb::conv_umma_multi_destroy(mu);
    if (v->scratch) cudaFree(v->scratch);
    delete v;
}

// Builds (once) what the instance needs to run batches of `nb` images: resolved parameters, input
// descriptors, scratch, grouped-launch tables and one executable graph per stage group.
int ensure_variant(pb_instance* in, int nb, Variant** out) {
    PB_REQUIRE(in && nb >= 1 && nb <= in->cap, "batch %d does not fit this instance (capacity %d)", nb, in ? in->cap : 0);
    if (in->variants[(size_t)nb - 1]) { *out = in->variants[(size_t)nb - 1]; return PB_OK; }
    pb_model* m = in->m;
    PB_CUDA(cudaSetDevice(m->device));
    Variant* v = new Variant();
    v->nb = nb;
    const size_t cap = (size_t)in->cap;
    // launch geometry and scratch layout of every stage at this batch
    std::vector<pb_launch_info> infos(m->stages.size());
    std::vector<size_t> scratch_off(m->stages.size(), 0);
    size_t scratch_bytes = 0;
    for (size_t i = 0; i < m->stages.size(); ++i) {
        const int rc = stage_info_batched(m, (int)i, nb, &infos[i]);
        if (rc != PB_OK) { destroy_variant(v); return rc; }
        if (infos[i].scratch_bytes) {
            scratch_off[i] = scratch_bytes;
            scratch_bytes += pb::round_up((size_t)infos[i].scratch_bytes, (size_t)256);
        }
    }
    cudaError_t e = cudaSuccess;
    if (scratch_bytes) {
        e = cudaMalloc((void**)&v->scratch, scratch_bytes);
        if (e == cudaSuccess) e = cudaMemset(v->scratch, 0, scratch_bytes);
        if (e != cudaSuccess) { destroy_variant(v); return pb::cuda_fail(e, "split-K scratch", __FILE__, __LINE__); }
    }
    v->params.resize(m->stages.size());
    v->xmaps.assign(m->stages.size(), nullptr);
    for (size_t i = 0; i < m->stages.size(); ++i) {
        const Stage& st = m->stages[i];
        pb_op_params p = st.p;
        p.batch = nb;
        p.x = st.x_is_input ? (const void*)in->in_dev : (const void*)(in->arena + cap * st.x_off);
        p.y = st.y_is_output ? (void*)in->out_dev : (void*)(in->arena + cap * st.y_off);
        p.residual = st.has_res ? (const void*)(in->arena + cap * st.res_off) : nullptr;
        p.scratch = infos[i].scratch_bytes ? v->scratch + scratch_off[i] : nullptr;
        p.scratch_bytes = infos[i].scratch_bytes;
        v->params[i] = p;
        if (st.kind == PB_STAGE_CONV_UMMA) {
            const int rc = pb::conv_umma_xmap_create(&p, &v->xmaps[i]);
            if (rc != PB_OK) { destroy_variant(v); return rc; }
        }
    }
    v->group_info.resize(m->groups.size());
    for (size_t g = 0; g < m->groups.size(); ++g) v->group_info[g] = group_footprint(m, (int)g, infos);
    v->graphs.assign(m->groups.size(), nullptr);
    v->multis.resize(m->groups.size());
    // descriptor tables of the launches that go through one (grouped convolutions; with the persistent kernel
    // every tensor-core convolution)
    for (size_t g = 0; g < m->groups.size(); ++g) {
        const pb_model::Group& grp = m->groups[g];
        v->multis[g].assign(grp.launches.size(), nullptr);
        for (size_t li = 0; li < grp.launches.size(); ++li) {
            const std::vector<int>& l = grp.launches[li];
            if (!uses_multi(m, l)) continue;
            std::vector<const pb::ConvUmmaPlan*> plans;
            std::vector<const pb::ConvUmmaXMap*> xm;
            std::vector<const pb_op_params*> pp;
            std::vector<int> kinds;
            for (int s : l) { plans.push_back(m->stages[s].plan); xm.push_back(v->xmaps[s]); pp.push_back(&v->params[s]); kinds.push_back(m->stages[s].kind); }
            const int rc = pb::conv_umma_multi_create(plans.data(), xm.data(), pp.data(), kinds.data(), (int)l.size(), &v->multis[g][li]);
            if (rc != PB_OK) { destroy_variant(v); return rc; }
        }
    }
    // PB_GRAPH_SINGLE=0: single-kernel groups are launched as plain kernels (about 3 us more host time each)
    const bool single_graphs = env_flag("PB_GRAPH_SINGLE", true);
    bool any_graph = single_graphs && !m->groups.empty();
    for (const pb_model::Group& g : m->groups) any_graph = any_graph || g.count > 1;
    if (any_graph) {
        (void)pb::device_error_flag_ptr(m->device);      // allocate it now: nothing may allocate during capture
        cudaStream_t cap_stream;
        e = cudaStreamCreateWithFlags(&cap_stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { destroy_variant(v); return pb::cuda_fail(e, "capture stream", __FILE__, __LINE__); }
        int rc = PB_OK;
        const bool pdl = env_flag("PB_PDL", true);
        const bool parallel = env_flag("PB_GRAPH_BRANCHES", false);
        for (size_t g = 0; rc == PB_OK && g < m->groups.size(); ++g) {
            const pb_model::Group& grp = m->groups[g];
            if (grp.count <= 1 && !single_graphs) continue;
            if (parallel && !m->fuse_branches) {
                rc = capture_group(in, *v, (int)g, cap_stream, pdl, true);
                if (rc == PB_OK) continue;
                cudaGetLastError();                   // a driver that cannot capture this: the chain below
            }
            rc = capture_group_chain(in, *v, (int)g, cap_stream, pdl);
            if (rc != PB_OK && pdl) {                 // a driver that cannot capture programmatic edges: plain edges
                cudaGetLastError();
                rc = capture_group_chain(in, *v, (int)g, cap_stream, false);
            }
        }
        cudaStreamDestroy(cap_stream);
        if (rc != PB_OK) { destroy_variant(v); return rc; }
    }
    in->variants[(size_t)nb - 1] = v;
    *out = v;
    return PB_OK;
}

}  // namespace

extern "C" {

int pb_op_info(int kind, const pb_op_params* p, pb_launch_info* out) {
    PB_REQUIRE(p && out, "pb_op_info: NULL argument");
    if (kind == PB_STAGE_CONV_UMMA) return pb::conv_umma_info(p, out);
    if (kind == PB_STAGE_MNIST_FUSED) return pb::mnist_fused_info(out);
    return pb::simple_op_info(kind, p, out);
}

int pb_op_launch(int kind, const pb_op_params* p, void* stream, uint32_t job_id, void* notifier) {
    PB_REQUIRE(p != nullptr, "pb_op_launch: NULL params");
    if (kind == PB_STAGE_CONV_UMMA) return pb::conv_umma_launch(p, (cudaStream_t)stream, job_id, notifier);
    return pb::simple_op_launch(kind, p, (cudaStream_t)stream, job_id, notifier);
}

int64_t pb_op_pack_weights(int kind, const pb_op_params* p, const float* w_oihw, void* dst_host) {
    if (!p || !w_oihw) { pb::set_error("pb_op_pack_weights: NULL argument"); return PB_ERR_INVALID; }
    if (kind == PB_STAGE_CONV_UMMA) return pb::conv_umma_pack_weights(p, w_oihw, dst_host);
    return pb::simple_pack_weights(kind, p, w_oihw, dst_host);
}

int pb_conv_umma_time(const pb_op_params* p, int mode, int iters, size_t flush_bytes, double* us_out) { return pb::conv_umma_time(p, mode, iters, flush_bytes, us_out); }

void pb_set_conv_split_gain_us(double us) { pb::conv_umma_set_split_gain_us(us); }

int pb_conv_umma_supported(const pb_op_params* p) { return p && pb::conv_umma_supported(p) ? 1 : 0; }

int pb_conv2d_umma_noalloc(const pb_op_params* p, void* stream, uint32_t job_id, void* notifier) {
    return pb::conv_umma_launch_noalloc(p, (cudaStream_t)stream, job_id, notifier);
}

int pb_model_load(const char* pack_path, int device, int precision, pb_model** out) {
    PB_REQUIRE(pack_path && out, "pb_model_load: NULL argument");
    FILE* f = fopen(pack_path, "rb");
    if (!f) { pb::set_error("cannot open model pack %s", pack_path); return PB_ERR_IO; }
    fseek(f, 0, SEEK_END);
    const long fsize = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> data((size_t)(fsize > 0 ? fsize : 0));
    const size_t got = fsize > 0 ? fread(data.data(), 1, data.size(), f) : 0;
    fclose(f);
    if (got != data.size() || data.size() < 64 || memcmp(data.data(), "PB2PACK\0", 8) != 0) {
        pb::set_error("%s is not a model pack", pack_path);
        return PB_ERR_IO;
    }
    uint32_t hdr[6];
    memcpy(hdr, data.data() + 8, sizeof(hdr));
    uint64_t n_floats;
    memcpy(&n_floats, data.data() + 32, 8);
    const uint32_t version = hdr[0], nt = hdr[1], no = hdr[2], t_in = hdr[3], t_out = hdr[4], hint = hdr[5];
    const size_t need = 64 + (size_t)nt * 16 + (size_t)no * (96 + 64) + (size_t)n_floats * 4;
    if (version != 1 || need != data.size() || t_in >= nt || t_out >= nt) {
        pb::set_error("%s: malformed pack (version %u, %zu bytes, expected %zu)", pack_path, version, data.size(), need);
        return PB_ERR_IO;
    }
    PB_CUDA(cudaSetDevice(device));

    pb_model* m = new pb_model();
    m->device = device;
    m->dtype = precision < 0 ? (int)hint : precision;
    m->name = std::string((const char*)data.data() + 40, strnlen((const char*)data.data() + 40, 24));
    m->t_in = (int)t_in;
    m->t_out = (int)t_out;
    const int vec = m->dtype == 0 ? 4 : 8;
    const size_t es = m->dtype == 0 ? 4 : 2;

    const uint8_t* pt = data.data() + 64;
    for (uint32_t i = 0; i < nt; ++i) {
        uint32_t rec[4];
        memcpy(rec, pt + 16 * i, 16);
        TensorInfo ti;
        ti.C = (int)rec[0]; ti.H = (int)rec[1]; ti.W = (int)rec[2];
        ti.Cs = pb::round_up(ti.C, vec);
        ti.bytes = pb::round_up((size_t)ti.H * ti.W * ti.Cs * es, (size_t)256);
        ti.offset = m->arena_bytes;
        if ((int)i != m->t_out) m->arena_bytes += ti.bytes;
        m->tensors.push_back(ti);
    }
    std::vector<PackOp> ops(no);
    memcpy(ops.data(), pt + 16 * (size_t)nt, (size_t)no * 96);
    const uint8_t* pn = pt + 16 * (size_t)nt + 96 * (size_t)no;
    const float* W = reinterpret_cast<const float*>(pn + 64 * (size_t)no);
    m->in_floats = (size_t)m->tensors[t_in].C * m->tensors[t_in].H * m->tensors[t_in].W;
    m->out_floats = (size_t)m->tensors[t_out].C * m->tensors[t_out].H * m->tensors[t_out].W;

#define PB_FAIL_LOAD(rc_)            \
    do {                             \
        int rc2_ = (rc_);            \
        if (rc2_ != PB_OK) {         \
            pb_model_destroy(m);     \
            return rc2_;             \
        }                            \
    } while (0)

    // ---- MNIST in one kernel (fp32 only) ----
    if (m->dtype == 0 && env_flag("PB_FUSE_MNIST", true) && is_mnist_topology(ops, m->tensors, m->t_in)) {
        m->mnist_fused = true;
        auto woff = [](const PackOp& o) { return ((uint64_t)o.w_off_hi << 32) | o.w_off_lo; };
        auto boff = [](const PackOp& o) { return ((uint64_t)o.b_off_hi << 32) | o.b_off_lo; };
        std::vector<float> w1(200), w2(3200), wd(2560);
        const float* s1 = W + woff(ops[0]);   // [8][1][5][5]
        for (int k = 0; k < 8; ++k) for (int t = 0; t < 25; ++t) w1[t * 8 + k] = s1[k * 25 + t];
        const float* s2 = W + woff(ops[2]);   // [16][8][5][5]
        for (int k = 0; k < 16; ++k) for (int c = 0; c < 8; ++c) for (int t = 0; t < 25; ++t) w2[(t * 8 + c) * 16 + k] = s2[(k * 8 + c) * 25 + t];
        const float* sd = W + woff(ops[4]);   // [10][16*4*4] in (c, h, w) order -> (h, w, c)
        for (int o = 0; o < 10; ++o) for (int c = 0; c < 16; ++c) for (int hw = 0; hw < 16; ++hw) wd[o * 256 + hw * 16 + c] = sd[o * 256 + c * 16 + hw];
        PB_FAIL_LOAD(upload(m, w1.data(), 800, (void**)&m->w1));
        PB_FAIL_LOAD(upload(m, W + boff(ops[0]), 32, (void**)&m->b1));
        PB_FAIL_LOAD(upload(m, w2.data(), 12800, (void**)&m->w2));
        PB_FAIL_LOAD(upload(m, W + boff(ops[2]), 64, (void**)&m->b2));
        PB_FAIL_LOAD(upload(m, wd.data(), 10240, (void**)&m->wd));
        PB_FAIL_LOAD(upload(m, W + boff(ops[4]), 40, (void**)&m->bd));
        Stage st{};
        st.kind = PB_STAGE_MNIST_FUSED;
        st.name = "mnist_fused";
        st.x_is_input = true; st.y_is_output = true; st.has_res = false;
        st.out_tensor = m->t_out;
        memset(&st.p, 0, sizeof(st.p));
        pb::mnist_fused_info(&st.info);
        m->stages.push_back(st);
        build_groups(m);
        *out = m;
        return PB_OK;
    }

    const bool use_umma = m->dtype == 1 && !env_flag("PB_DISABLE_UMMA", false);

    // ---- patch-matrix lowering of the stem ----
    // When the model input (<= 4 channels) feeds exactly one dense convolution and the tensor-core path is
    // on, stage 0 writes that convolution's im2col rows instead of a channels-last image and the
    // convolution runs pointwise over R*S*C channels (PB_PATCH_INPUT=0 turns this off).
    int patch_op = -1, patch_tensor = -1;
    if (use_umma && env_flag("PB_PATCH_INPUT", true) && m->tensors[t_in].C <= 4) {
        int readers = 0, first = -1;
        for (uint32_t i = 0; i < no; ++i) {
            if (ops[i].in0 == t_in || ops[i].in1 == t_in) { ++readers; if (first < 0) first = (int)i; }
        }
        if (readers == 1 && ops[first].type == OP_CONV && ops[first].in0 == t_in && ops[first].in1 == kNone &&
            (ops[first].groups == 0 || ops[first].groups == 1) && ops[first].r * ops[first].s > 1 && ops[first].out < nt &&
            ops[first].dil_h <= 1 && ops[first].dil_w <= 1 &&
            ops[first].cout % 8 == 0 && ops[first].out_c_off % 8 == 0 && (int)ops[first].out != m->t_out) {   // = what the tensor-core path needs
            patch_op = first;
            const PackOp& o = ops[first];
            const TensorInfo& ty = m->tensors[o.out];
            TensorInfo tp;
            tp.C = (int)(o.r * o.s) * m->tensors[t_in].C; tp.H = ty.H; tp.W = ty.W;
            tp.Cs = pb::round_up(tp.C, vec);
            tp.bytes = pb::round_up((size_t)tp.H * tp.W * tp.Cs * es, (size_t)256);
            tp.offset = m->arena_bytes;
            m->arena_bytes += tp.bytes;
            patch_tensor = (int)m->tensors.size();
            m->tensors.push_back(tp);
        }
    }

    // ---- stage 0: NCHW fp32 -> channels-last image, or -> patch matrix ----
    {
        Stage st{};
        st.kind = PB_STAGE_INPUT;
        const TensorInfo& ti = m->tensors[t_in];
        memset(&st.p, 0, sizeof(st.p));
        st.p.dtype = m->dtype; st.p.C = ti.C; st.p.H = ti.H; st.p.W = ti.W; st.p.Cs = ti.C;
        st.x_is_input = true; st.y_is_output = false; st.has_res = false;
        if (patch_op >= 0) {
            const PackOp& o = ops[patch_op];
            const TensorInfo& tp = m->tensors[patch_tensor];
            st.name = "input_patches";
            st.p.K = tp.C; st.p.P = tp.H; st.p.Q = tp.W; st.p.Ks = tp.Cs;
            st.p.R = (int)o.r; st.p.S = (int)o.s; st.p.stride_h = (int)o.stride_h; st.p.stride_w = (int)o.stride_w;
            st.p.pad_h = (int)o.pad_h; st.p.pad_w = (int)o.pad_w;
            st.y_off = tp.offset;
            st.out_tensor = patch_tensor;
        } else {
            st.name = "input_layout";
            st.p.K = ti.C; st.p.P = ti.H; st.p.Q = ti.W; st.p.Ks = ti.Cs;
            st.y_off = ti.offset;
            st.out_tensor = (int)t_in;
        }
        PB_FAIL_LOAD(pb::simple_op_info(st.kind, &st.p, &st.info));
        m->stages.push_back(st);
    }

    for (uint32_t i = 0; i < no; ++i) {
        const PackOp& o = ops[i];
        if (o.in0 >= nt || o.out >= nt || (o.in1 != kNone && o.in1 >= nt)) {
            pb::set_error("%s: op %u references a missing tensor", pack_path, i);
            PB_FAIL_LOAD(PB_ERR_IO);
        }
        const TensorInfo& tx = m->tensors[o.in0];
        const TensorInfo& ty = m->tensors[o.out];
        const uint64_t w_off = ((uint64_t)o.w_off_hi << 32) | o.w_off_lo;
        const uint64_t b_off = ((uint64_t)o.b_off_hi << 32) | o.b_off_lo;
        Stage st{};
        st.name = std::string((const char*)pn + 64 * i, strnlen((const char*)pn + 64 * i, 64));
        st.out_tensor = (int)o.out;
        st.in_tensor = (int)o.in0;
        st.res_tensor = o.in1 != kNone ? (int)o.in1 : -1;
        pb_op_params& p = st.p;
        memset(&p, 0, sizeof(p));
        p.dtype = m->dtype;
        p.C = tx.C; p.H = tx.H; p.W = tx.W; p.Cs = tx.Cs;
        p.K = (int)o.cout; p.P = ty.H; p.Q = ty.W; p.Ks = ty.Cs;
        p.out_c_off = (int)o.out_c_off;
        p.R = (int)o.r; p.S = (int)o.s; p.stride_h = (int)o.stride_h; p.stride_w = (int)o.stride_w;
        p.pad_h = (int)o.pad_h; p.pad_w = (int)o.pad_w; p.groups = (int)(o.groups ? o.groups : 1);
        p.act = (int)o.act; p.flags = (int)(o.flags & 1);
        p.dil_h = o.dil_h > 1 ? (int)o.dil_h : 1; p.dil_w = o.dil_w > 1 ? (int)o.dil_w : 1;
        st.x_is_input = false;
        st.x_off = tx.offset;
        st.y_is_output = (int)o.out == m->t_out;
        st.y_off = ty.offset;
        st.has_res = o.in1 != kNone;
        if (st.has_res) { st.res_off = m->tensors[o.in1].offset; p.res_Cs = m->tensors[o.in1].Cs; p.residual = (const void*)1; }
        if (st.y_is_output) p.flags |= 2;

        std::vector<uint8_t> packed;
        switch (o.type) {
            case OP_CONV: {
                if (st.y_is_output) { pb::set_error("a convolution cannot write the fp32 model output"); PB_FAIL_LOAD(PB_ERR_INVALID); }
                std::vector<float> w_patch;
                const float* w_src = W + w_off;
                if ((int)i == patch_op) {
                    // pointwise over the patch matrix: input channel k = (r*S + s)*C + c, weights reordered to match
                    const TensorInfo& tp = m->tensors[patch_tensor];
                    const int C0 = tx.C, R0 = (int)o.r, S0 = (int)o.s;
                    w_patch.resize((size_t)p.K * tp.C);
                    for (int k = 0; k < p.K; ++k)
                        for (int c = 0; c < C0; ++c)
                            for (int r = 0; r < R0; ++r)
                                for (int s2 = 0; s2 < S0; ++s2)
                                    w_patch[(size_t)k * tp.C + (size_t)(r * S0 + s2) * C0 + c] = w_src[(((size_t)k * C0 + c) * R0 + r) * S0 + s2];
                    w_src = w_patch.data();
                    p.C = tp.C; p.H = tp.H; p.W = tp.W; p.Cs = tp.Cs;
                    p.R = p.S = 1; p.stride_h = p.stride_w = 1; p.pad_h = p.pad_w = 0;
                    st.x_off = tp.offset;
                    st.in_tensor = patch_tensor;
                }
                const bool dw = p.groups > 1 && p.groups == p.C && p.K == p.C;
                if (dw && (p.dil_h > 1 || p.dil_w > 1)) { pb::set_error("%s: dilated depthwise convolution is not supported", pack_path); PB_FAIL_LOAD(PB_ERR_INVALID); }
                if (dw) st.kind = PB_STAGE_DWCONV;
                else if (use_umma && pb::conv_umma_supported(&p)) st.kind = PB_STAGE_CONV_UMMA;
                else st.kind = PB_STAGE_CONV_SIMT;
                // UMMA sees the padded channel stride as its input-channel count; SIMT uses the real one.
                if ((int)i == patch_op && st.kind != PB_STAGE_CONV_UMMA) {
                    pb::set_error("%s: the stem convolution does not fit the tensor-core path after patch lowering", pack_path);
                    PB_FAIL_LOAD(PB_ERR_INVALID);
                }
                const int64_t nbytes = pb_op_pack_weights(st.kind, &p, w_src, nullptr);
                if (nbytes < 0) PB_FAIL_LOAD((int)nbytes);
                packed.resize((size_t)nbytes);
                pb_op_pack_weights(st.kind, &p, w_src, packed.data());
                PB_FAIL_LOAD(upload(m, packed.data(), packed.size(), &st.w_dev));
                if (p.act == 3 && dw) { pb::set_error("%s: PReLU on a depthwise convolution is not supported", pack_path); PB_FAIL_LOAD(PB_ERR_INVALID); }
                PB_FAIL_LOAD(upload(m, W + b_off, (size_t)p.K * 4 * (p.act == 3 ? 2 : 1), (void**)&st.bias_dev));   // PReLU: [bias | slope]
                break;
            }
            case OP_DENSE: {
                st.kind = PB_STAGE_DENSE;
                // input is [H][W][Cs] on the device; boundary weights are [K][C*H*W] in (c, h, w) order
                const int n_dev = tx.H * tx.W * tx.Cs;
                packed.assign((size_t)p.K * n_dev * (m->dtype == 0 ? 4 : 2), 0);
                const float* src = W + w_off;
                for (int k = 0; k < p.K; ++k)
                    for (int c = 0; c < tx.C; ++c)
                        for (int hw = 0; hw < tx.H * tx.W; ++hw)
                            pb::store_elem(packed.data(), (size_t)k * n_dev + (size_t)hw * tx.Cs + c,
                                           src[(size_t)k * o.cin + (size_t)c * tx.H * tx.W + hw], m->dtype);
                p.C = n_dev; p.H = 1; p.W = 1; p.Cs = n_dev;
                PB_FAIL_LOAD(upload(m, packed.data(), packed.size(), &st.w_dev));
                PB_FAIL_LOAD(upload(m, W + b_off, (size_t)p.K * 4, (void**)&st.bias_dev));
                break;
            }
            case OP_MAXPOOL:
            case OP_AVGPOOL:
                st.kind = o.type == OP_MAXPOOL ? PB_STAGE_MAXPOOL : PB_STAGE_AVGPOOL;
                p.K = tx.C;
                if (o.flags & 8) {      // a per-channel bias is added to the pooled value (then p.act applies)
                    if (b_off + (uint64_t)tx.C > n_floats) { pb::set_error("%s: pooling op %u: bias outside the weights", pack_path, i); PB_FAIL_LOAD(PB_ERR_IO); }
                    PB_FAIL_LOAD(upload(m, W + b_off, (size_t)tx.C * 4, (void**)&st.bias_dev));
                }
                break;
            case OP_GAP: st.kind = PB_STAGE_GAP; p.K = tx.C; break;
            case OP_ADD: st.kind = PB_STAGE_ADD; break;
            case OP_AFFINE: {
                // reads the first `cin` channels of its input tensor (a prefix of a concatenation)
                if (o.cin == 0 || (int)o.cin > tx.C || o.cout != o.cin) { pb::set_error("%s: affine op %u has bad channel counts", pack_path, i); PB_FAIL_LOAD(PB_ERR_INVALID); }
                st.kind = PB_STAGE_AFFINE;
                p.C = (int)o.cin; p.K = (int)o.cin;
                PB_FAIL_LOAD(upload(m, W + w_off, (size_t)p.C * 4, &st.w_dev));
                PB_FAIL_LOAD(upload(m, W + b_off, (size_t)p.C * 4, (void**)&st.bias_dev));
                break;
            }
            case OP_SOFTMAX: st.kind = PB_STAGE_SOFTMAX; p.C = tx.C * tx.H * tx.W; break;
            case OP_DETECT: {
                // cin = anchors per cell, cout = priors of the whole model, out_c_off = first prior of this map;
                // weights = this map's priors [H*W*anchors][4], bias block = {centre variance, size variance}
                const uint64_t n_here = (uint64_t)tx.H * tx.W * o.cin;
                if (o.cin == 0 || tx.C != (int)(6 * o.cin) || !st.y_is_output || (uint64_t)ty.C * ty.H * ty.W != 6ull * o.cout ||
                    (uint64_t)o.out_c_off + n_here > o.cout || w_off + 4 * n_here > n_floats || b_off + 2 > n_floats) {
                    pb::set_error("%s: detection head %u does not fit its tensors", pack_path, i);
                    PB_FAIL_LOAD(PB_ERR_INVALID);
                }
                st.kind = PB_STAGE_DETECT;
                PB_FAIL_LOAD(upload(m, W + w_off, (size_t)n_here * 16, &st.w_dev));
                PB_FAIL_LOAD(upload(m, W + b_off, 8, (void**)&st.bias_dev));
                break;
            }
            default:
                pb::set_error("%s: unknown operator type %u", pack_path, o.type);
                PB_FAIL_LOAD(PB_ERR_IO);
        }
        if (st.y_is_output && !(st.kind == PB_STAGE_DENSE || st.kind == PB_STAGE_GAP || st.kind == PB_STAGE_SOFTMAX || st.kind == PB_STAGE_DETECT)) {
            pb::set_error("stage kind %d cannot write the fp32 model output", st.kind);
            PB_FAIL_LOAD(PB_ERR_INVALID);
        }
        p.w = st.w_dev;
        p.bias = st.bias_dev;
        // every instance brings scratch memory of the model's largest requirement: size the launch for it
        p.scratch = (void*)16;
        p.scratch_bytes = ~0ull;
        PB_FAIL_LOAD(pb_op_info(st.kind, &p, &st.info));
        if (st.info.scratch_bytes) {
            st.scratch_off = m->scratch_bytes;
            m->scratch_bytes += pb::round_up((size_t)st.info.scratch_bytes, (size_t)256);
        }
        if (st.kind == PB_STAGE_CONV_UMMA) PB_FAIL_LOAD(pb::conv_umma_plan_create(&p, st.w_dev, &st.plan));
        m->stages.push_back(st);
    }
#undef PB_FAIL_LOAD
    build_groups(m);
    *out = m;
    return PB_OK;
}

void pb_model_destroy(pb_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    for (auto& st : m->stages) if (st.plan) pb::conv_umma_plan_destroy(st.plan);
    for (void* d : m->allocs) cudaFree(d);
    delete m;
}

size_t pb_model_input_bytes(const pb_model* m) { return m ? m->in_floats * 4 : 0; }
size_t pb_model_output_bytes(const pb_model* m) { return m ? m->out_floats * 4 : 0; }
int pb_model_num_stages(const pb_model* m) { return m ? (int)m->stages.size() : 0; }

int pb_model_stage_info(const pb_model* m, int stage, pb_launch_info* out) {
    PB_REQUIRE(m && out && stage >= 0 && stage < (int)m->stages.size(), "pb_model_stage_info: bad stage %d", stage);
    *out = m->stages[stage].info;
    return PB_OK;
}

const char* pb_model_stage_name(const pb_model* m, int stage) {
    if (!m || stage < 0 || stage >= (int)m->stages.size()) return "";
    return m->stages[stage].name.c_str();
}

int pb_instance_create_batched(pb_model* m, int capacity, int prepare_all, pb_instance** out) {
    PB_REQUIRE(m && out, "pb_instance_create: NULL argument");
    PB_REQUIRE(capacity >= 1 && capacity <= pb::kMaxGang, "pb_instance_create: capacity %d outside 1..%d", capacity, pb::kMaxGang);
    PB_CUDA(cudaSetDevice(m->device));
    pb_instance* in = new pb_instance();
    in->m = m;
    in->cap = capacity;
    in->variants.assign((size_t)capacity, nullptr);
    const size_t cap = (size_t)capacity;
    const size_t in_bytes = pb::round_up(cap * m->in_floats * 4, (size_t)256), out_bytes = pb::round_up(cap * m->out_floats * 4, (size_t)256);
    cudaError_t e = cudaMalloc((void**)&in->arena, cap * m->arena_bytes + 256);
    if (e == cudaSuccess) e = cudaMemset(in->arena, 0, cap * m->arena_bytes + 256);
    if (e == cudaSuccess) e = cudaMalloc((void**)&in->in_dev, in_bytes);
    if (e == cudaSuccess) e = cudaMemset(in->in_dev, 0, in_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&in->out_dev, out_bytes);
    if (e == cudaSuccess) e = cudaMemset(in->out_dev, 0, out_bytes);
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&in->slot_host, sizeof(pb::LaunchSlot), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaMalloc((void**)&in->slot_dev, sizeof(pb::LaunchSlot));
    if (e != cudaSuccess) {
        pb_instance_destroy(in);
        return pb::cuda_fail(e, "instance buffers", __FILE__, __LINE__);
    }
    memset(in->slot_host, 0, sizeof(pb::LaunchSlot));
    for (int nb = 1; nb <= (prepare_all ? capacity : 1); ++nb) {
        Variant* v = nullptr;
        const int rc = ensure_variant(in, nb, &v);
        if (rc != PB_OK) { pb_instance_destroy(in); return rc; }
    }
    *out = in;
    return PB_OK;
}

int pb_instance_create(pb_model* m, pb_instance** out) { return pb_instance_create_batched(m, 1, 1, out); }

int pb_instance_capacity(const pb_instance* in) { return in ? in->cap : 0; }

void pb_instance_destroy(pb_instance* in) {
    if (!in) return;
    if (in->m) cudaSetDevice(in->m->device);
    for (Variant* v : in->variants) destroy_variant(v);
    if (in->slot_host) cudaFreeHost(in->slot_host);
    if (in->slot_dev) cudaFree(in->slot_dev);
    if (in->arena) cudaFree(in->arena);
    if (in->in_dev) cudaFree(in->in_dev);
    if (in->out_dev) cudaFree(in->out_dev);
    delete in;
}

void* pb_instance_input_dev(pb_instance* in) { return in ? in->in_dev : nullptr; }
void* pb_instance_output_dev(pb_instance* in) { return in ? in->out_dev : nullptr; }

static int launch_stage_batched(pb_instance* in, int stage, int nb, void* stream, uint32_t job_id, void* notifier) {
    PB_REQUIRE(in && stage >= 0 && stage < (int)in->m->stages.size(), "pb_instance_launch_stage: bad stage %d", stage);
    Variant* v = nullptr;
    const int rc = ensure_variant(in, nb, &v);
    if (rc != PB_OK) return rc;
    return launch_stage_with(in, *v, stage, &v->params[stage], (cudaStream_t)stream, job_id, notifier, in->in_dev, in->out_dev);
}

int pb_instance_launch_stage(pb_instance* in, int stage, void* stream, uint32_t job_id, void* notifier) {
    return launch_stage_batched(in, stage, 1, stream, job_id, notifier);
}

int pb_model_num_groups(const pb_model* m) { return m ? (int)m->groups.size() : 0; }

int pb_model_group_info(const pb_model* m, int group, pb_launch_info* out) {
    PB_REQUIRE(m && out && group >= 0 && group < (int)m->groups.size(), "pb_model_group_info: bad group %d", group);
    *out = m->groups[group].info;
    return PB_OK;
}

int pb_model_group_info_batched(const pb_model* m, int group, int batch, pb_launch_info* out) {
    PB_REQUIRE(m && out && group >= 0 && group < (int)m->groups.size(), "pb_model_group_info_batched: bad group %d", group);
    PB_REQUIRE(batch >= 1 && batch <= pb::kMaxGang, "pb_model_group_info_batched: batch %d outside 1..%d", batch, pb::kMaxGang);
    std::vector<pb_launch_info> infos(m->stages.size());
    const pb_model::Group& g = m->groups[(size_t)group];
    for (int i = g.first; i < g.first + g.count; ++i) {
        const int rc = stage_info_batched(m, i, batch, &infos[(size_t)i]);
        if (rc != PB_OK) return rc;
    }
    *out = group_footprint(m, group, infos);
    return PB_OK;
}

int pb_model_stage_info_batched(const pb_model* m, int stage, int batch, pb_launch_info* out) {
    PB_REQUIRE(m && out && stage >= 0 && stage < (int)m->stages.size(), "pb_model_stage_info_batched: bad stage %d", stage);
    PB_REQUIRE(batch >= 1 && batch <= pb::kMaxGang, "pb_model_stage_info_batched: batch %d outside 1..%d", batch, pb::kMaxGang);
    return stage_info_batched(m, stage, batch, out);
}

int pb_model_group_stages(const pb_model* m, int group, int* first, int* count) {
    PB_REQUIRE(m && group >= 0 && group < (int)m->groups.size(), "pb_model_group_stages: bad group %d", group);
    if (first) *first = m->groups[group].first;
    if (count) *count = m->groups[group].count;
    return PB_OK;
}

int pb_model_group_plan(const pb_model* m, int group, int32_t* stage_order, int32_t* launch_index, int max_stages) {
    PB_REQUIRE(m && stage_order && launch_index && group >= 0 && group < (int)m->groups.size(), "pb_model_group_plan: bad argument (group %d)", group);
    int n = 0;
    const pb_model::Group& g = m->groups[group];
    for (size_t li = 0; li < g.launches.size(); ++li)
        for (int s : g.launches[li]) {
            if (n >= max_stages) return n;
            stage_order[n] = s;
            launch_index[n] = (int32_t)li;
            ++n;
        }
    return n;
}

int pb_instance_launch_group_batched(pb_instance* in, int group, int batch, void* stream, uint32_t job_id, void* notifier,
                                     const void* const* io_in, void* const* io_out) {
    PB_REQUIRE(in && group >= 0 && group < (int)in->m->groups.size(), "pb_instance_launch_group: bad group %d", group);
    Variant* v = nullptr;
    const int vrc = ensure_variant(in, batch, &v);
    if (vrc != PB_OK) return vrc;
    const pb_model* m = in->m;
    const pb_model::Group& g = m->groups[group];
    pb::LaunchSlot* s = in->slot_host;
    s->nf = static_cast<llis::job::FinishedBlockNotifier*>(notifier);
    s->job_id = job_id;
    for (int i = 0; i < batch; ++i) {
        s->io_in[i] = (io_in && io_in[i]) ? static_cast<const float*>(io_in[i]) : in->in_dev + (size_t)i * m->in_floats;
        s->io_out[i] = (io_out && io_out[i]) ? static_cast<float*>(io_out[i]) : in->out_dev + (size_t)i * m->out_floats;
    }
    if (v->graphs[group]) {
        PB_CUDA(cudaGraphLaunch(v->graphs[group], (cudaStream_t)stream));
        return PB_OK;
    }
    // single kernel, no graph: a direct launch
    const int stage = g.first;
    if (v->multis[(size_t)group][0])
        return pb::conv_umma_multi_launch(v->multis[(size_t)group][0], (cudaStream_t)stream, job_id, notifier, false);
    pb_op_params p = v->params[stage];
    if (batch == 1) {
        if (stage == 0) p.x = s->io_in[0];
        if (m->stages[stage].y_is_output) p.y = s->io_out[0];
        return launch_stage_with(in, *v, stage, &p, (cudaStream_t)stream, job_id, notifier, s->io_in[0], s->io_out[0]);
    }
    // a batch's buffers are not one array: the kernel takes them, and the notifier, from the pinned slot
    if (stage == 0) p.x = nullptr;
    if (m->stages[stage].y_is_output) p.y = nullptr;
    return launch_stage_with(in, *v, stage, &p, (cudaStream_t)stream, pb::kSlotNotify, in->slot_host, nullptr, nullptr);
}

int pb_instance_launch_group(pb_instance* in, int group, void* stream, uint32_t job_id, void* notifier, const void* io_in,
                             void* io_out) {
    const void* ins[1] = {io_in};
    void* outs[1] = {io_out};
    return pb_instance_launch_group_batched(in, group, 1, stream, job_id, notifier, ins, outs);
}

// H2D of `batch` inputs, the model (group by group as CUDA graphs, or kernel by kernel), D2H of the outputs.
static int run_sync(pb_instance* in, int batch, bool by_groups, const float* input_host, float* output_host) {
    PB_REQUIRE(in && input_host && output_host, "pb_instance_run_sync: NULL argument");
    PB_REQUIRE(batch >= 1 && batch <= in->cap, "pb_instance_run_sync: batch %d does not fit capacity %d", batch, in->cap);
    pb_model* m = in->m;
    PB_CUDA(cudaSetDevice(m->device));
    cudaStream_t st;
    PB_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    int rc = PB_OK;
    cudaError_t e = cudaMemcpyAsync(in->in_dev, input_host, (size_t)batch * m->in_floats * 4, cudaMemcpyHostToDevice, st);
    if (by_groups) {
        for (int g = 0; e == cudaSuccess && rc == PB_OK && g < (int)m->groups.size(); ++g)
            rc = pb_instance_launch_group_batched(in, g, batch, st, 0, nullptr, nullptr, nullptr);
    } else {
        for (int i = 0; e == cudaSuccess && rc == PB_OK && i < (int)m->stages.size(); ++i) rc = launch_stage_batched(in, i, batch, st, 0, nullptr);
    }
    if (e == cudaSuccess && rc == PB_OK) e = cudaMemcpyAsync(output_host, in->out_dev, (size_t)batch * m->out_floats * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && rc == PB_OK) e = cudaStreamSynchronize(st);
    cudaStreamDestroy(st);
    if (rc != PB_OK) return rc;
    if (e != cudaSuccess) return pb::cuda_fail(e, "pb_instance_run_sync", __FILE__, __LINE__);
    return PB_OK;
}

int pb_instance_run_groups_sync(pb_instance* in, const float* input_host, float* output_host) { return run_sync(in, 1, true, input_host, output_host); }
int pb_instance_run_sync(pb_instance* in, const float* input_host, float* output_host) { return run_sync(in, 1, false, input_host, output_host); }
int pb_instance_run_batch_sync(pb_instance* in, int batch, int by_groups, const float* inputs_host, float* outputs_host) {
    return run_sync(in, batch, by_groups != 0, inputs_host, outputs_host);
}

int pb_instance_read_tensor(pb_instance* in, int tensor, float* dst, size_t dst_floats) {
    PB_REQUIRE(in && dst && tensor >= 0 && tensor < (int)in->m->tensors.size(), "pb_instance_read_tensor: bad tensor %d", tensor);
    pb_model* m = in->m;
    const TensorInfo& t = m->tensors[tensor];
    const size_t n = (size_t)t.C * t.H * t.W;
    PB_REQUIRE(dst_floats >= n, "pb_instance_read_tensor: destination too small");
    PB_CUDA(cudaSetDevice(m->device));
    PB_CUDA(cudaDeviceSynchronize());
    if (tensor == m->t_out) {
        PB_CUDA(cudaMemcpy(dst, in->out_dev, n * 4, cudaMemcpyDeviceToHost));
        return PB_OK;
    }
    if (m->mnist_fused) { pb::set_error("intermediate tensors do not exist in the fused MNIST kernel"); return PB_ERR_INVALID; }
    const size_t es = m->dtype == 0 ? 4 : 2;
    std::vector<uint8_t> raw((size_t)t.H * t.W * t.Cs * es);
    PB_CUDA(cudaMemcpy(raw.data(), in->arena + (size_t)in->cap * t.offset, raw.size(), cudaMemcpyDeviceToHost));   // image 0
    for (int c = 0; c < t.C; ++c)
        for (int hw = 0; hw < t.H * t.W; ++hw) {
            const size_t s = (size_t)hw * t.Cs + c;
            float v;
            if (m->dtype == 0) v = reinterpret_cast<const float*>(raw.data())[s];
            else { uint32_t u = (uint32_t)reinterpret_cast<const uint16_t*>(raw.data())[s] << 16; memcpy(&v, &u, 4); }
            dst[(size_t)c * t.H * t.W + hw] = v;
        }
    return PB_OK;
}

int pb_instance_stage_params(pb_instance* in, int stage, int batch, pb_op_params* out) {
    PB_REQUIRE(in && out && stage >= 0 && stage < (int)in->m->stages.size(), "pb_instance_stage_params: bad stage %d", stage);
    Variant* v = nullptr;
    const int rc = ensure_variant(in, batch, &v);
    if (rc != PB_OK) return rc;
    *out = v->params[(size_t)stage];
    return PB_OK;
}

int pb_instance_time_stage_batched(pb_instance* in, int stage, int batch, int iters, size_t flush_bytes, double* us_out) {
    PB_REQUIRE(in && us_out && iters > 0 && stage >= 0 && stage < (int)in->m->stages.size(), "pb_instance_time_stage: bad arguments");
    PB_CUDA(cudaSetDevice(in->m->device));
    cudaStream_t st;
    PB_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    void* flush = nullptr;
    if (flush_bytes) PB_CUDA(cudaMalloc(&flush, flush_bytes));
    cudaEvent_t e0, e1;
    PB_CUDA(cudaEventCreate(&e0));
    PB_CUDA(cudaEventCreate(&e1));
    int rc = PB_OK;
    double total_ms = 0;
    for (int i = 0; i < 3 && rc == PB_OK; ++i) rc = launch_stage_batched(in, stage, batch, st, 0, nullptr);   // warm-up
    for (int i = 0; i < iters && rc == PB_OK; ++i) {
        if (flush) cudaMemsetAsync(flush, i & 0xff, flush_bytes, st);
        cudaEventRecord(e0, st);
        rc = launch_stage_batched(in, stage, batch, st, 0, nullptr);
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) { rc = PB_ERR_CUDA; pb::set_error("timing run failed: %s", cudaGetErrorString(cudaGetLastError())); break; }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        total_ms += ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (flush) cudaFree(flush);
    cudaStreamDestroy(st);
    if (rc != PB_OK) return rc;
    *us_out = total_ms * 1000.0 / iters;
    return PB_OK;
}

int pb_instance_time_stage(pb_instance* in, int stage, int iters, size_t flush_bytes, double* us_out) {
    return pb_instance_time_stage_batched(in, stage, 1, iters, flush_bytes, us_out);
}

}  // extern "C"
