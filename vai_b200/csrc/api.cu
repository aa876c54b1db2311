// C ABI of the backend (include/vaicu.h): device, buffers, streams, and the
// Linear plan — the shape -> kernel choice that vAi makes in Linear::prepare()
// (vai/nodes/linear.h:2291-2704) and the launches it records in Linear::run()
// (linear.h:2706-2798).  Nothing here falls back to the CPU.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "common.cuh"
#include "tc_gemm.h"

using namespace vaicu;

struct vaicu_device {
    int ordinal;
    int sm_count;
    int cc_major, cc_minor;
    int* status_word;   // device memory; kernels set it when a bounded wait expires
};
struct vaicu_buffer {
    void* ptr;
    size_t bytes;
    int ordinal;
};
struct vaicu_graph {
    cudaGraphExec_t exec;
};
struct vaicu_event {
    cudaEvent_t ev;
};

namespace {

thread_local char g_last_error[256] = {0};

int cuda_fail(cudaError_t e, const char* what)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ? VAICU_ERR_NO_DEVICE : VAICU_ERR_CUDA;
}
#define VAICU_CUDA(call)                                              \
    do {                                                              \
        cudaError_t e__ = (call);                                     \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call);         \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved at run time so that the library carries no
// link-time dependency on libcuda (it must load on machines without a driver).
EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// [rows, K] row-major 16-bit matrix, boxes of box_rows x 64 elements, 128-byte swizzle.
int encode_map(CUtensorMap* map, const void* base, int dtype, uint32_t rows, uint32_t K, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) { snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled unavailable"); return VAICU_ERR_CUDA; }
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2u};
    const cuuint32_t box[2] = {64u, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(map, dtype == VAICU_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                          2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled failed (%d)", (int)r);
        return VAICU_ERR_CUDA;
    }
    return VAICU_OK;
}

bool valid_dtype(int d) { return d == VAICU_DTYPE_F32 || d == VAICU_DTYPE_F16 || d == VAICU_DTYPE_BF16; }
bool is16(int d) { return d == VAICU_DTYPE_F16 || d == VAICU_DTYPE_BF16; }
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1u) / b; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

namespace vaicu {
void set_last_error(const char* where, const char* what)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", where ? where : "", what ? what : "");
}
}  // namespace vaicu

struct vaicu_linear_plan {
    vaicu_device* dev;
    vaicu_linear_desc d;
    vaicu_linear_tuning tune;   // the caller's overrides (all "library's choice" for a plain plan)
    int kernel;               // VAICU_KERNEL_*
    // GEMV
    GemvConfig gemv_vec, gemv_any;
    // FMA tile (also the fallback of the tensor-core plans)
    FmaTileConfig fma;
    bool fma_partial;
    size_t fma_ws_bytes;
    // tensor-core GEMM
    bool tc, tc_swap, tc_cast;
    TcParams tcp;
    int tc_grid;
    size_t tc_smem;
    size_t ws_cast_bytes, ws_partial_bytes;
    // TMA descriptors are made on first use of a base pointer and kept: two per operand, so that a caller
    // that alternates two activation (or weight) buffers re-encodes nothing after the first two runs.
    // map_b_tail: the weights with the strip box of the tail round.
    CUtensorMap map_a[2], map_b[2], map_b_tail[2];
    const void* map_a_base[2];
    const void* map_b_base[2];
    uint32_t map_a_next, map_b_next;
    size_t workspace_bytes;
    uint32_t launches;
    // split-K on the single-CTA tensor-core kernel: finished-splits count per tile, owned by the plan
    // (all zero between launches), so that the fold needs no launch of its own
    unsigned int* tile_done;
    // what the most recent run on this plan enqueued (VAICU_KERNEL_*), and whether it was the
    // 16-byte-vector form of that kernel: differs from `kernel` when a view's alignment sent
    // the call to a fallback
    int last_kernel, last_vectorized;
    // this plan as the first member of a group on the tensor-core kernel (vaicu_linear_run_group)
    struct GroupState* group;
};

// Two or three plans on the swapped tensor-core kernel run as one Linear over their weights' rows
// side by side: the plan of that virtual Linear and the TMA descriptors of the members' tensors.
struct GroupState {
    const vaicu_linear_plan* members[3];
    int count;
    vaicu_linear_plan* virt;
    uint32_t rows[3];
    CUtensorMap maps_w[3];
    const void* w_base[3];
    CUtensorMap map_act[2];
    const void* act_base[2];
    uint32_t act_next;
};

namespace {

int validate_desc(const vaicu_linear_desc* d)
{
    if (!d) return VAICU_ERR_INVALID_VALUE;
    if (d->M == 0 || d->N == 0 || d->K == 0) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(d->i_dtype) || !valid_dtype(d->w_dtype) || !valid_dtype(d->o_dtype)) return VAICU_ERR_INVALID_VALUE;
    if (d->has_bias && !valid_dtype(d->b_dtype)) return VAICU_ERR_INVALID_VALUE;
    if (d->epilogue < 0 || d->epilogue > VAICU_EPILOGUE_SIGMOID) return VAICU_ERR_INVALID_VALUE;
    if (d->residual_order != 0 && d->residual_order != 1) return VAICU_ERR_INVALID_VALUE;
    if (d->split_size != 0 && d->split_size < 32) return VAICU_ERR_INVALID_VALUE;   // vAi linear.h:2442
    if ((uint64_t)d->M * d->N >= (1ull << 32)) return VAICU_ERR_INVALID_VALUE;       // vAi indexes with uint32
    const uint64_t out_elems = (uint64_t)d->M * (d->gate_fuse ? d->N / 2u : d->N);
    if (d->gate_fuse) {
        if (d->N % 2u) return VAICU_ERR_INVALID_VALUE;
        if (d->has_residual) return VAICU_ERR_UNSUPPORTED;
        if (d->has_bias && d->bias_elems != d->N && !(d->bias_elems == 0 && d->M == 1u))
            return VAICU_ERR_UNSUPPORTED;   // one bias per weight row
    }
    // broadcast rule of vAi linear.h:2333-2338: whole rows that tile O
    if (d->has_bias && d->bias_elems && !d->gate_fuse &&
        (d->bias_elems % d->N || ((uint64_t)d->M * d->N) % d->bias_elems)) return VAICU_ERR_INVALID_VALUE;
    if (d->has_residual && d->residual_elems && (d->residual_elems % d->N || out_elems % d->residual_elems))
        return VAICU_ERR_INVALID_VALUE;
    return VAICU_OK;
}

LinearArgs make_args(const vaicu_linear_desc& d, const void* I, const void* W, const void* bias, const void* res, void* O)
{
    LinearArgs a{};
    a.I = I; a.W = W; a.bias = bias; a.res = res; a.O = O;
    a.M = d.M; a.N = d.N; a.K = d.K;
    a.i_dtype = d.i_dtype; a.w_dtype = d.w_dtype; a.o_dtype = d.o_dtype; a.b_dtype = d.b_dtype;
    a.has_bias = d.has_bias ? 1 : 0; a.has_res = d.has_residual ? 1 : 0;
    a.residual_order = d.residual_order; a.epilogue = d.epilogue; a.gate_fuse = d.gate_fuse ? 1 : 0;
    a.bias_elems = d.has_bias ? d.bias_elems : 0; a.res_elems = d.has_residual ? d.residual_elems : 0;
    a.scale = d.scalar_scale;
    return a;
}

int operand_mode(bool present, uint32_t elems, uint32_t row_len)
{
    if (!present) return OPERAND_NONE;
    if (elems == 0) return OPERAND_FULL;
    if (elems == row_len) return OPERAND_PER_COLUMN;
    return OPERAND_MODULO;
}

// Split-K for the FMA tile kernel: the caller's span, else one span
// (vAi linear.h:2440-2450 resolves the same two cases).
void plan_fma(vaicu_linear_plan* pl)
{
    const vaicu_linear_desc& d = pl->d;
    uint32_t split_size = d.K, split_count = 1;
    if (d.split_size) {
        split_size = d.split_size < d.K ? d.split_size : d.K;
        split_count = ceil_div(d.K, split_size);
    } else {
        // Fewer tiles than two per SM: split K until there are about that many blocks (a block keeps
        // one trip of loads in flight, so an SM needs several to hide their latency), at least 256 of K each.
        // Measured on 128 x 768 x 3072 fp32 (96 tiles): 51 us unsplit, 39 / 29 / 31 us with 2 / 3 / 4 spans.
        const uint32_t tiles = ceil_div(d.M, 64u) * ceil_div(d.N, 64u);
        const uint32_t sms = (uint32_t)pl->dev->sm_count;
        if (tiles < 2u * sms && d.K >= 512u) {
            uint32_t want = ceil_div(2u * sms, tiles);
            if (want > 16u) want = 16u;
            split_size = (uint32_t)align_up(ceil_div(d.K, want), 64u);
            if (split_size < 256u) split_size = 256u;
            split_count = ceil_div(d.K, split_size);
        }
    }
    if (split_count > 65535u) { split_count = 65535u; split_size = ceil_div(d.K, split_count); split_count = ceil_div(d.K, split_size); }
    pl->fma.split_size = split_size;
    pl->fma.split_count = split_count;
    pl->fma_partial = split_count > 1u || d.gate_fuse;
    pl->fma_ws_bytes = pl->fma_partial ? (size_t)split_count * d.M * d.N * sizeof(float) : 0;
}

bool tc_eligible(const vaicu_linear_desc& d)
{
    if (!is16(d.w_dtype)) return false;
    if (!(d.i_dtype == d.w_dtype || d.i_dtype == VAICU_DTYPE_F32)) return false;
    if (d.K % 8u) return false;
    return true;
}

// Tile / split choice of the tensor-core kernel (the role selectLinearTile plays
// in the reference, vAi linear.h:2101-2119): fill the SMs with whole waves of
// the widest tile, and split K only when the tile grid cannot occupy them.
void plan_tc(vaicu_linear_plan* pl, bool swap)
{
    const vaicu_linear_desc& d = pl->d;
    const uint32_t sms = (uint32_t)pl->dev->sm_count;
    const bool gate = d.gate_fuse != 0;
    const uint32_t H = gate ? d.N / 2u : d.N;
    TcParams& t = pl->tcp;
    memset(&t, 0, sizeof(t));
    t.M = d.M; t.N = d.N; t.K = d.K; t.H = H;
    t.kblocks = ceil_div(d.K, 64u);
    t.grp_t1 = t.grp_t2 = kNoGroup;
    uint32_t bn;
    t.tile_rows = 128u;
    if (swap) {
        bn = (uint32_t)align_up(d.M, 16u);
        if (bn > 128u) bn = 128u;
        t.tiles_b = ceil_div(d.M, bn);
        // Weight rows per tile.  128 fills the MMA; but a layer with fewer 128-row tiles than SMs leaves
        // SMs without work, and a CTA streams its weights no faster than about one SM's share of the HBM
        // bandwidth.  Shorter tiles (the MMA still spans 128 rows, the rest of the slot is not loaded and
        // its lanes are not read) spread such a layer over all SMs without a K split and its fold.  Among the
        // heights that give more than half a tile per SM (fewer tiles are split along K below) and keep
        // the weights the larger part of what a CTA loads, pick the one with the fewest bytes per CTA:
        // rounds x (weight rows + activation rows) per k-block.
        const uint32_t boxes = gate ? 2u : 1u;
        uint32_t best_rows = 128u;
        uint64_t best_cost = ~0ull;
        for (uint32_t rows = 128u; rows >= 32u && !d.split_size; rows -= 8u) {
            if (boxes * rows < bn) break;
            const uint32_t tiles = ceil_div(H, rows) * t.tiles_b;
            if (tiles * 2u <= sms) continue;
            const uint64_t cost = (uint64_t)ceil_div(tiles, sms) * (boxes * rows + bn);
            if (cost < best_cost) { best_cost = cost; best_rows = rows; }
        }
        if (pl->tune.tc_tile_rows) best_rows = pl->tune.tc_tile_rows;
        t.tile_rows = best_rows;
        t.tiles_a = ceil_div(H, t.tile_rows);
    } else {
        // CTA pairs (cta_group::2): two neighbouring SMs share one 256-row tile and each
        // stages half of the weights' tile; both accumulator buffers stay in use.
        bool pair = d.M > 128u;
        if (pl->tune.tc_pair >= 0) pair = pl->tune.tc_pair != 0;
        // output columns per tile: bn (bn / 2 with gate)
        const uint32_t cand[3] = {256u, 128u, 64u};
        const uint32_t rows = pair ? 256u : 128u, units = pair ? sms / 2u : sms;
        double best = -1.0;
        bn = 256u;
        for (uint32_t c : cand) {
            const uint32_t out_cols = gate ? c / 2u : c;
            const uint32_t tiles = ceil_div(d.M, rows) * ceil_div(H, out_cols);
            const uint32_t waves = ceil_div(tiles, units);
            double eff = (double)tiles / ((double)waves * units);
            // narrower tiles re-read the activations more often and issue shorter MMAs
            // (measured on 8192 x 3072 x 3072: 1256 / 888 TFLOP/s for 256 / 128 on pairs)
            if (pair) eff *= (c == 256u) ? 1.0 : (c == 128u ? 0.70 : 0.45);
            else eff *= (c == 256u) ? 1.0 : (c == 128u ? 0.88 : 0.70);
            // a tile wider than the whole output is wasted work
            if (out_cols > (uint32_t)align_up(H, 16u) && c != 64u) eff *= (double)H / out_cols;
            if (eff > best) { best = eff; bn = c; }
        }
        if (pl->tune.tc_bn) bn = pl->tune.tc_bn;   // validated when the plan was created
        // Single-CTA alternative for 256-row tiles: two A boxes per stage and two MMAs per
        // k-step; needs all 512 TMEM columns at bn = 256 (no epilogue overlap).
        bool wide = !pair && bn == 256u && d.M >= 512u &&
                    ceil_div(d.M, 256u) * ceil_div(H, gate ? bn / 2u : bn) * 100u >= 85u * sms;
        if (pl->tune.tc_wide >= 0) wide = pl->tune.tc_wide != 0 && bn * 2u <= 512u && !pair;
        t.pair = pair ? 1u : 0u;
        t.wide = wide ? 1u : 0u;
        t.tiles_a = ceil_div(d.M, (wide || pair) ? 256u : 128u);
        t.tiles_b = ceil_div(H, gate ? bn / 2u : bn);
    }
    t.bn = bn;
    t.num_tiles = t.tiles_a * t.tiles_b;
    t.group = t.tiles_a < 16u ? t.tiles_a : 16u;
    // split-K
    const uint32_t units = t.pair ? sms / 2u : sms;      // tiles that run at the same time
    uint32_t kb_per_split = t.kblocks;
    if (d.split_size) {
        kb_per_split = ceil_div(d.split_size, 64u);
    } else if (t.num_tiles * 2u <= units && t.kblocks >= 8u) {
        uint32_t want = units / t.num_tiles;
        const uint32_t max_splits = t.kblocks / 4u;      // at least 4 k-blocks (256 of K) per split
        if (want > max_splits) want = max_splits;
        if (want > 32u) want = 32u;
        if (want >= 2u) kb_per_split = ceil_div(t.kblocks, want);
    }
    if (pl->tune.tc_splits && !d.split_size) kb_per_split = ceil_div(t.kblocks, pl->tune.tc_splits);
    if (kb_per_split == 0u) kb_per_split = 1u;
    if (kb_per_split > t.kblocks) kb_per_split = t.kblocks;
    t.kb_per_split = kb_per_split;
    t.splits = ceil_div(t.kblocks, kb_per_split);
    // descriptor: fp32 accumulate, A/B formats, both K-major, N >> 3, M >> 4
    const uint32_t fmt = d.w_dtype == VAICU_DTYPE_BF16 ? 1u : 0u;
    t.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((bn >> 3) << 17) | (((t.pair ? 256u : 128u) >> 4) << 24);
    const uint32_t a_boxes = ((gate && swap) || t.wide) ? 2u : 1u;
    const uint32_t a_bytes = a_boxes * 128u * 128u;
    const uint32_t stage_bytes = a_bytes + (t.pair ? bn / 2u : bn) * 128u;      // per CTA
    auto size_ring = [&](uint32_t extra) {
        uint32_t stages = (uint32_t)((kTcMaxSmem - 2048u - extra) / stage_bytes);
        if (stages > 8u) stages = 8u;
        // A CTA of the swapped kernel that streams only a few k-blocks (a K split of a small layer) gets a
        // ring of four stages: two such CTAs then fit on an SM, so the next launch's CTAs set up and request
        // their weights while this launch's finish (q / o of a 4B-class model at batch 64: 8.3 -> 7.7 us and
        // 8.8 -> 8.1 us; layers with long K ranges lose with the short ring and keep the deep one).
        if (swap && t.splits > 1u && t.kb_per_split <= 10u && stages > 4u) stages = 4u;
        if (pl->tune.tc_stages && pl->tune.tc_stages < stages) stages = pl->tune.tc_stages;
        t.stages = stages;
        pl->tc_smem = (size_t)stages * stage_bytes + 1024u + 256u + extra;
    };
    size_ring(0u);
    // Split-K folded inside clusters (swapped kernel), on request (tc_fold = 3): the S splits of a tile run as
    // one cluster and add their accumulators up through distributed shared memory, so neither the fp32
    // partial sums nor the fold launch exist.  S is 2, 4 or 8 (each CTA finishes bn / S activation rows, a
    // multiple of 16) and all clusters must be resident at once.  Not the default: measured on B200 the two
    // cluster barriers and the remote reads take as long as the dependent fold launch they replace (q of a
    // 4B-class model at batch 64: 8.1 us either way), and the fold launch handles bias / residual with far
    // more threads (attention output + residual: 12.6 us in clusters, 8.7 us with the fold launch).
    t.cfold = 0u;
    if (swap && !gate && t.splits > 1u && !d.split_size && pl->tune.tc_fold == 3) {
        const uint64_t per_kb = (uint64_t)t.tile_rows * 128u + bn * 128u;      // bytes a CTA loads per k-block
        uint32_t best = 0u;
        uint64_t best_cost = ~0ull;
        for (uint32_t S = 8u; S >= 2u; S /= 2u) {
            if (bn % S || (bn / S) % 16u) continue;
            if (pl->tune.tc_splits && pl->tune.tc_splits != S) continue;      // the caller's split count stands
            const uint32_t kbs = ceil_div(t.kblocks, S);
            if (kbs < 2u || ceil_div(t.kblocks, kbs) != S) continue;
            if (t.num_tiles * S > sms) continue;
            const uint64_t cost = (uint64_t)kbs * per_kb + 32u * 1024u;
            if (cost < best_cost) { best_cost = cost; best = S; }
        }
        if (best) {
            const uint32_t keep_kb = t.kb_per_split, keep_splits = t.splits;
            t.cfold = best;
            t.splits = best;
            t.kb_per_split = ceil_div(t.kblocks, best);
            size_ring(bn * 128u * 4u);
            int clusters = 0;
            if (t.stages < 2u || tc_swap_max_clusters(pl->tc_smem, best, &clusters) != cudaSuccess || (uint32_t)clusters < t.num_tiles) {
                cudaGetLastError();
                t.cfold = 0u;
                t.splits = keep_splits;
                t.kb_per_split = keep_kb;
                size_ring(0u);
            }
        }
    }
    const uint32_t acc_cols = a_boxes * bn;
    t.acc_bufs = 2u * acc_cols <= 512u ? 2u : 1u;
    uint32_t cols = 32u;
    while (cols < t.acc_bufs * acc_cols) cols *= 2u;
    t.tmem_cols = cols;
    t.o_dtype = d.o_dtype; t.b_dtype = d.b_dtype; t.epilogue = d.epilogue; t.residual_order = d.residual_order;
    t.has_bias = d.has_bias ? 1 : 0; t.has_res = d.has_residual ? 1 : 0; t.gate = gate ? 1 : 0;
    t.bias_mode = operand_mode(d.has_bias != 0, d.bias_elems, d.N);
    t.res_mode = operand_mode(d.has_residual != 0, d.residual_elems, H);
    t.bias_elems = d.bias_elems; t.res_elems = d.residual_elems;
    t.scale = d.scalar_scale;
    t.status = pl->dev->status_word;
    const uint32_t work = t.num_tiles * t.splits;
    pl->tc_grid = (int)((work < sms || t.cfold) ? work : sms);      // cluster fold: one work item per CTA
    if (t.pair) {
        int clusters = 0;
        if (tc_pair_max_clusters(pl->tc_smem, &clusters) != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            clusters = (int)(sms / 2u);
        }
        if ((uint32_t)clusters > work) clusters = (int)work;
        pl->tc_grid = 2 * clusters;
    }
    // Last round of the CTA-pair kernel: when the tile count leaves a partial round (384 tiles on 74
    // clusters: 5 full rounds and 14 tiles), those tiles are cut into column strips so that the round is
    // shorter and keeps more clusters busy: as many strips per tile (2 or 4) as there are clusters for.
    t.tail_first = t.num_tiles;
    t.tail_split = 1u;
    t.idesc_tail = t.idesc;
    if (t.pair && t.splits == 1u && pl->tune.tc_tail_strips != 1) {
        const uint32_t clusters = (uint32_t)pl->tc_grid / 2u;
        const uint32_t rem = clusters ? t.num_tiles % clusters : 0u;
        uint32_t strips = 1u;
        if (rem && t.num_tiles > clusters) {
            for (uint32_t c = 2u; c <= 4u; c *= 2u) {
                const uint32_t width = bn / c;
                if (bn % c || width % 32u || rem * c > clusters) continue;
                strips = c;
            }
        }
        if (pl->tune.tc_tail_strips > 1) {
            const uint32_t c = (uint32_t)pl->tune.tc_tail_strips;
            strips = (rem && bn % c == 0u && (bn / c) % 32u == 0u) ? c : 1u;
        }
        if (strips > 1u) {
            t.tail_first = t.num_tiles - rem;
            t.tail_split = strips;
            const uint32_t fmt2 = d.w_dtype == VAICU_DTYPE_BF16 ? 1u : 0u;
            t.idesc_tail = (1u << 4) | (fmt2 << 7) | (fmt2 << 10) | (((bn / strips) >> 3) << 17) | ((256u >> 4) << 24);
        }
    }
    pl->tc_swap = swap;
    pl->tc_cast = d.i_dtype == VAICU_DTYPE_F32;
    pl->ws_cast_bytes = pl->tc_cast ? align_up((size_t)d.M * d.K * 2u, 256u) : 0;
    pl->ws_partial_bytes = (t.splits > 1u && !t.cfold) ? (size_t)t.splits * d.M * d.N * sizeof(float) : 0;
}

vaicu_linear_tuning default_tuning()
{
    vaicu_linear_tuning t;
    memset(&t, 0, sizeof(t));
    t.tc_pair = t.tc_wide = -1;
    return t;
}

int validate_tuning(const vaicu_linear_tuning& t)
{
    if (t.kernel != 0 && (t.kernel < VAICU_KERNEL_GEMV || t.kernel > VAICU_KERNEL_TC_SKINNY)) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_pair < -1 || t.tc_pair > 1 || t.tc_wide < -1 || t.tc_wide > 1) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_bn && (t.tc_bn < 16u || t.tc_bn > 256u || t.tc_bn % 16u)) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_splits > 1024u) return VAICU_ERR_INVALID_VALUE;
    if (t.gemv_rows != 0 && t.gemv_rows != 2 && t.gemv_rows != 4) return VAICU_ERR_INVALID_VALUE;
    const int k = t.gemv_k_warps;
    if (k != 0 && k != 1 && k != 2 && k != 4 && k != 8) return VAICU_ERR_INVALID_VALUE;
    if (t.gemv_unroll != 0 && t.gemv_unroll != 2 && t.gemv_unroll != 4) return VAICU_ERR_INVALID_VALUE;
    if (t.gemv_grid < 0) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_fold < 0 || t.tc_fold > 3) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_stages == 1u || t.tc_stages > 8u) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_tile_rows && (t.tc_tile_rows < 8u || t.tc_tile_rows > 128u || t.tc_tile_rows % 8u)) return VAICU_ERR_INVALID_VALUE;
    if (t.tc_tail_strips != 0 && t.tc_tail_strips != 1 && t.tc_tail_strips != 2 && t.tc_tail_strips != 4) return VAICU_ERR_INVALID_VALUE;
    return VAICU_OK;
}

int build_plan(vaicu_device* dev, const vaicu_linear_desc* desc, const vaicu_linear_tuning& tuning, vaicu_linear_plan** out)
{
    if (!dev || !out) return VAICU_ERR_INVALID_VALUE;
    int rc = validate_desc(desc);
    if (rc != VAICU_OK) return rc;
    rc = validate_tuning(tuning);
    if (rc != VAICU_OK) return rc;
    const int force_kernel = tuning.kernel;
    vaicu_linear_plan* pl = new (std::nothrow) vaicu_linear_plan();
    if (!pl) return VAICU_ERR_INVALID_VALUE;
    pl->dev = dev;
    pl->d = *desc;
    pl->tune = tuning;
    pl->tile_done = nullptr;
    pl->group = nullptr;
    if (!pl->d.has_bias) { pl->d.bias_elems = 0; pl->d.b_dtype = VAICU_DTYPE_NONE; }
    if (!pl->d.has_residual) pl->d.residual_elems = 0;
    // a [N] bias under M == 1 "covers O" (elems 0); name it per-row so every kernel takes the cheap index
    if (pl->d.has_bias && pl->d.bias_elems == 0 && pl->d.M == 1u) pl->d.bias_elems = pl->d.N;
    const vaicu_linear_desc& d = pl->d;
    LinearArgs a = make_args(d, nullptr, nullptr, nullptr, nullptr, nullptr);
    pl->gemv_vec = choose_gemv(a, dev->sm_count, true, &pl->tune);
    pl->gemv_any = choose_gemv(a, dev->sm_count, false, &pl->tune);
    plan_fma(pl);
    pl->tc = false;
    int kernel = force_kernel;
    if (kernel == 0) {
        // Few rows: the weight-streaming kernel (vAi useSlabPath takes M <= 8,
        // linear.h:320).  Measured on B200 the FMA kernel stops being memory-bound past
        // M = 4 (shared-memory reads of the activations), while the swapped tensor-core
        // kernel streams weights at full rate for any M, so M = 5..8 go there when the
        // operands allow it.
        if (d.M <= 4u || (d.M <= 8u && !tc_eligible(d))) kernel = VAICU_KERNEL_GEMV;
        else if (tc_eligible(d)) kernel = d.M <= 128u ? VAICU_KERNEL_TC_SKINNY : VAICU_KERNEL_TC_GEMM;
        else kernel = VAICU_KERNEL_FMA_TILE;
    }
    switch (kernel) {
    case VAICU_KERNEL_GEMV:
        if (d.M > 8u) { delete pl; return VAICU_ERR_UNSUPPORTED; }
        pl->workspace_bytes = 0;
        pl->launches = 1;
        break;
    case VAICU_KERNEL_FMA_TILE:
        pl->workspace_bytes = pl->fma_ws_bytes;
        pl->launches = pl->fma_partial ? 2 : 1;
        break;
    case VAICU_KERNEL_TC_GEMM:
    case VAICU_KERNEL_TC_SKINNY:
        if (!tc_eligible(d) || (kernel == VAICU_KERNEL_TC_SKINNY && d.M > 256u)) { delete pl; return VAICU_ERR_UNSUPPORTED; }
        pl->tc = true;
        plan_tc(pl, kernel == VAICU_KERNEL_TC_SKINNY);
        pl->workspace_bytes = pl->ws_cast_bytes + pl->ws_partial_bytes;
        // unaligned operands fall back to the FMA tile kernel at run time
        if (pl->fma_ws_bytes > pl->workspace_bytes) pl->workspace_bytes = pl->fma_ws_bytes;
        if (pl->tcp.splits > 1u && !pl->tcp.pair && pl->tune.tc_fold == 1) {
            // the CTAs of a tile's splits fold it together: a counter per tile, device state that lives with the plan
            const size_t bytes = align_up((size_t)pl->tcp.num_tiles * sizeof(unsigned int), 256u);
            cudaError_t e = cudaSetDevice(dev->ordinal);
            if (e == cudaSuccess) e = cudaMalloc(&pl->tile_done, bytes);
            if (e == cudaSuccess) e = cudaMemset(pl->tile_done, 0, bytes);
            if (e != cudaSuccess) {
                if (pl->tile_done) cudaFree(pl->tile_done);
                delete pl;
                return cuda_fail(e, "split-K tile counters");
            }
        }
        pl->launches = 1u + (pl->tc_cast ? 1u : 0u) + ((pl->tcp.splits > 1u && !pl->tile_done && !pl->tcp.cfold) ? 1u : 0u);
        break;
    default:
        delete pl;
        return VAICU_ERR_INVALID_VALUE;
    }
    pl->kernel = kernel;
    pl->last_kernel = 0;
    pl->last_vectorized = 0;
    pl->map_a_base[0] = pl->map_a_base[1] = pl->map_b_base[0] = pl->map_b_base[1] = nullptr;
    pl->map_a_next = pl->map_b_next = 0u;
    *out = pl;
    return VAICU_OK;
}

int run_fma(vaicu_linear_plan* pl, const LinearArgs& a, void* workspace, cudaStream_t s)
{
    if (pl->fma_partial && !workspace) return VAICU_ERR_WORKSPACE;
    float* partial = pl->fma_partial ? reinterpret_cast<float*>(workspace) : nullptr;
    VAICU_CUDA(launch_fma_tile(a, pl->fma, partial, s));
    if (partial) VAICU_CUDA(launch_splitk_reduce(a, partial, pl->fma.split_count, s));
    return VAICU_OK;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int vaicu_device_open(int ordinal, vaicu_device** out)
{
    if (!out) return VAICU_ERR_INVALID_VALUE;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
    if (ordinal < 0 || ordinal >= count) return VAICU_ERR_NO_DEVICE;
    cudaDeviceProp prop;
    VAICU_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10) {
        snprintf(g_last_error, sizeof(g_last_error), "device %d is sm_%d%d; this library holds sm_100a code only", ordinal,
                 prop.major, prop.minor);
        return VAICU_ERR_NO_DEVICE;
    }
    VAICU_CUDA(cudaSetDevice(ordinal));
    vaicu_device* d = new (std::nothrow) vaicu_device();
    if (!d) return VAICU_ERR_INVALID_VALUE;
    d->ordinal = ordinal;
    d->sm_count = prop.multiProcessorCount;
    d->cc_major = prop.major;
    d->cc_minor = prop.minor;
    e = cudaMalloc(&d->status_word, 256);
    if (e != cudaSuccess) { delete d; return cuda_fail(e, "cudaMalloc(status)"); }
    e = cudaMemset(d->status_word, 0, 256);
    if (e != cudaSuccess) { cudaFree(d->status_word); delete d; return cuda_fail(e, "cudaMemset(status)"); }
    *out = d;
    return VAICU_OK;
}

int vaicu_device_close(vaicu_device* dev)
{
    if (!dev) return VAICU_ERR_INVALID_VALUE;
    cudaSetDevice(dev->ordinal);
    cudaFree(dev->status_word);
    delete dev;
    return VAICU_OK;
}

int vaicu_device_sm_count(const vaicu_device* dev, int* out)
{
    if (!dev || !out) return VAICU_ERR_INVALID_VALUE;
    *out = dev->sm_count;
    return VAICU_OK;
}

int vaicu_device_synchronize(vaicu_device* dev)
{
    if (!dev) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaSetDevice(dev->ordinal));
    VAICU_CUDA(cudaDeviceSynchronize());
    return VAICU_OK;
}

int vaicu_device_status(vaicu_device* dev, int* out)
{
    if (!dev || !out) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaSetDevice(dev->ordinal));
    VAICU_CUDA(cudaDeviceSynchronize());
    int word = 0;
    VAICU_CUDA(cudaMemcpy(&word, dev->status_word, sizeof(int), cudaMemcpyDeviceToHost));
    *out = word;
    if (word) {
        VAICU_CUDA(cudaMemset(dev->status_word, 0, sizeof(int)));
        return VAICU_ERR_TIMEOUT;
    }
    return VAICU_OK;
}

int vaicu_device_selftest_wait_expiry(vaicu_device* dev, vaicu_stream_t stream)
{
    if (!dev) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaSetDevice(dev->ordinal));
    VAICU_CUDA(launch_wait_expiry_selftest(dev->status_word, (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_buffer_alloc(vaicu_device* dev, size_t bytes, vaicu_buffer** out)
{
    if (!dev || !out) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaSetDevice(dev->ordinal));
    vaicu_buffer* b = new (std::nothrow) vaicu_buffer();
    if (!b) return VAICU_ERR_INVALID_VALUE;
    // sizes round up to 4 bytes as in vAi's pool (vai/engine/buffer-pool.h:84); never 0
    b->bytes = bytes ? align_up(bytes, 4) : 4;
    b->ordinal = dev->ordinal;
    cudaError_t e = cudaMalloc(&b->ptr, b->bytes);
    if (e != cudaSuccess) { delete b; return cuda_fail(e, "cudaMalloc"); }
    *out = b;
    return VAICU_OK;
}

int vaicu_buffer_free(vaicu_buffer* buf)
{
    if (!buf) return VAICU_ERR_INVALID_VALUE;
    cudaSetDevice(buf->ordinal);
    cudaError_t e = cudaFree(buf->ptr);
    delete buf;
    if (e != cudaSuccess) return cuda_fail(e, "cudaFree");
    return VAICU_OK;
}

void* vaicu_buffer_ptr(const vaicu_buffer* buf) { return buf ? buf->ptr : nullptr; }
size_t vaicu_buffer_size(const vaicu_buffer* buf) { return buf ? buf->bytes : 0; }

int vaicu_memcpy_h2d(void* dst, const void* src, size_t bytes, vaicu_stream_t stream)
{
    if ((!dst || !src) && bytes) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return VAICU_OK;
}
int vaicu_memcpy_d2h(void* dst, const void* src, size_t bytes, vaicu_stream_t stream)
{
    if ((!dst || !src) && bytes) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return VAICU_OK;
}
int vaicu_memset(void* dst, int value, size_t bytes, vaicu_stream_t stream)
{
    if (!dst && bytes) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return VAICU_OK;
}
int vaicu_host_alloc_pinned(size_t bytes, void** out)
{
    if (!out) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaMallocHost(out, bytes ? bytes : 4));
    return VAICU_OK;
}
int vaicu_host_free_pinned(void* p)
{
    if (!p) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaFreeHost(p));
    return VAICU_OK;
}

int vaicu_stream_create(vaicu_device* dev, vaicu_stream_t* out)
{
    if (!dev || !out) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaSetDevice(dev->ordinal));
    cudaStream_t s;
    VAICU_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = (vaicu_stream_t)s;
    return VAICU_OK;
}
int vaicu_stream_sync(vaicu_stream_t stream)
{
    VAICU_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return VAICU_OK;
}
int vaicu_stream_destroy(vaicu_stream_t stream)
{
    if (!stream) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaStreamDestroy((cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_stream_wait_stream(vaicu_stream_t waiter, vaicu_stream_t signaler)
{
    if (!waiter || !signaler) return VAICU_ERR_INVALID_VALUE;
    cudaEvent_t e;
    VAICU_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    cudaError_t rc = cudaEventRecord(e, (cudaStream_t)signaler);
    if (rc == cudaSuccess) rc = cudaStreamWaitEvent((cudaStream_t)waiter, e, 0);
    cudaEventDestroy(e);   // released once the recorded work has completed
    if (rc != cudaSuccess) return cuda_fail(rc, "vaicu_stream_wait_stream");
    return VAICU_OK;
}

int vaicu_event_create(vaicu_event** out)
{
    if (!out) return VAICU_ERR_INVALID_VALUE;
    cudaEvent_t e;
    VAICU_CUDA(cudaEventCreate(&e));
    vaicu_event* r = new (std::nothrow) vaicu_event();
    if (!r) { cudaEventDestroy(e); return VAICU_ERR_INVALID_VALUE; }
    r->ev = e;
    *out = r;
    return VAICU_OK;
}
int vaicu_event_record(vaicu_event* ev, vaicu_stream_t stream)
{
    if (!ev) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaEventRecord(ev->ev, (cudaStream_t)stream));
    return VAICU_OK;
}
int vaicu_event_synchronize(vaicu_event* ev)
{
    if (!ev) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaEventSynchronize(ev->ev));
    return VAICU_OK;
}
int vaicu_event_elapsed_ms(vaicu_event* start, vaicu_event* stop, float* out_ms)
{
    if (!start || !stop || !out_ms) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaEventElapsedTime(out_ms, start->ev, stop->ev));
    return VAICU_OK;
}
int vaicu_event_destroy(vaicu_event* ev)
{
    if (!ev) return VAICU_ERR_INVALID_VALUE;
    cudaEventDestroy(ev->ev);
    delete ev;
    return VAICU_OK;
}

int vaicu_graph_capture_begin(vaicu_stream_t stream)
{
    if (!stream) return VAICU_ERR_INVALID_VALUE;   // the legacy default stream cannot be captured
    // Relaxed: other work of the host (e.g. a buffer of an older net being freed by a
    // destructor) must not invalidate the recording.
    VAICU_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeRelaxed));
    return VAICU_OK;
}
int vaicu_graph_capture_end(vaicu_stream_t stream, vaicu_graph** out)
{
    if (!stream || !out) return VAICU_ERR_INVALID_VALUE;
    cudaGraph_t g = nullptr;
    VAICU_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    vaicu_graph* r = new (std::nothrow) vaicu_graph();
    if (!r) { cudaGraphExecDestroy(exec); return VAICU_ERR_INVALID_VALUE; }
    r->exec = exec;
    *out = r;
    return VAICU_OK;
}
int vaicu_graph_launch(vaicu_graph* graph, vaicu_stream_t stream)
{
    if (!graph) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaGraphLaunch(graph->exec, (cudaStream_t)stream));
    return VAICU_OK;
}
int vaicu_graph_destroy(vaicu_graph* graph)
{
    if (!graph) return VAICU_ERR_INVALID_VALUE;
    cudaGraphExecDestroy(graph->exec);
    delete graph;
    return VAICU_OK;
}

int vaicu_linear_plan_create(vaicu_device* dev, const vaicu_linear_desc* desc, vaicu_linear_plan** out)
{
    return build_plan(dev, desc, default_tuning(), out);
}
int vaicu_linear_plan_create_forced(vaicu_device* dev, const vaicu_linear_desc* desc, int kernel, vaicu_linear_plan** out)
{
    if (kernel < VAICU_KERNEL_GEMV || kernel > VAICU_KERNEL_TC_SKINNY) return VAICU_ERR_INVALID_VALUE;
    vaicu_linear_tuning t = default_tuning();
    t.kernel = kernel;
    return build_plan(dev, desc, t, out);
}
int vaicu_linear_plan_create_tuned(vaicu_device* dev, const vaicu_linear_desc* desc, const vaicu_linear_tuning* tuning,
                                   vaicu_linear_plan** out)
{
    if (!tuning) return VAICU_ERR_INVALID_VALUE;
    return build_plan(dev, desc, *tuning, out);
}
int vaicu_linear_plan_destroy(vaicu_linear_plan* plan)
{
    if (!plan) return VAICU_ERR_INVALID_VALUE;
    if (plan->tile_done) {
        cudaSetDevice(plan->dev->ordinal);
        cudaFree(plan->tile_done);
    }
    if (plan->group) {
        vaicu_linear_plan_destroy(plan->group->virt);
        delete plan->group;
    }
    delete plan;
    return VAICU_OK;
}
int vaicu_linear_plan_info(const vaicu_linear_plan* plan, vaicu_linear_info* out)
{
    if (!plan || !out) return VAICU_ERR_INVALID_VALUE;
    memset(out, 0, sizeof(*out));
    out->kernel = plan->kernel;
    out->launches = plan->launches;
    out->workspace_bytes = plan->workspace_bytes;
    out->split_count = 1;
    if (plan->kernel == VAICU_KERNEL_FMA_TILE) {
        out->split_count = plan->fma.split_count; out->tile_m = 64; out->tile_n = 64;
    } else if (plan->tc) {
        out->split_count = plan->tcp.splits;
        const uint32_t outc = (plan->tcp.gate && !plan->tc_swap) ? plan->tcp.bn / 2u : plan->tcp.bn;
        out->tile_m = plan->tc_swap ? outc : ((plan->tcp.wide || plan->tcp.pair) ? 256u : 128u);
        out->tile_n = plan->tc_swap ? plan->tcp.tile_rows : outc;
    }
    return VAICU_OK;
}
int vaicu_linear_plan_last_run(const vaicu_linear_plan* plan, int* kernel, int* vectorized)
{
    if (!plan || !kernel || !vectorized) return VAICU_ERR_INVALID_VALUE;
    *kernel = plan->last_kernel;
    *vectorized = plan->last_vectorized;
    return VAICU_OK;
}
int vaicu_linear_workspace_bytes(const vaicu_linear_plan* plan, size_t* out)
{
    if (!plan || !out) return VAICU_ERR_INVALID_VALUE;
    *out = plan->workspace_bytes;
    return VAICU_OK;
}

namespace {
// Where the output goes: one dense buffer (n_dst == 1, ldo = width of O, col0 = 0), or the
// same column slab inside several wider buffers.
struct OutputSpec {
    uint32_t n_dst, ldo, col0;
    void* dst[8];
    uint32_t rs_rows, rs_slot;      // row-parallel run: rows per owner (0 = off) and this rank's slab in the owners' staging
};
int run_impl(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W, const void* bias,
             const void* residual, void* O, void* workspace, const OutputSpec* spec);
}  // namespace

int vaicu_linear_run(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W, const void* bias,
                     const void* residual, void* O, void* workspace)
{
    return run_impl(pl, stream, I, W, bias, residual, O, workspace, nullptr);
}

int vaicu_linear_run_reduce_scatter(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W,
                                    void* const* dsts, int n_dst, int slot, void* workspace)
{
    if (!pl || !dsts || n_dst < 1 || n_dst > 8 || slot < 0 || slot >= n_dst) return VAICU_ERR_INVALID_VALUE;
    const vaicu_linear_desc& d = pl->d;
    // partial sums only: anything after the dot product belongs to the fold that follows the exchange
    if (!pl->tc || pl->tcp.splits > 1u || d.has_residual || d.has_bias || d.gate_fuse || d.epilogue != VAICU_EPILOGUE_NONE ||
        d.scalar_scale != 1.0f)
        return VAICU_ERR_UNSUPPORTED;
    if (d.M % (uint32_t)n_dst) return VAICU_ERR_INVALID_VALUE;
    OutputSpec spec{};
    spec.n_dst = (uint32_t)n_dst;
    spec.ldo = d.N;
    spec.col0 = 0;
    spec.rs_rows = d.M / (uint32_t)n_dst;
    spec.rs_slot = (uint32_t)slot;
    for (int i = 0; i < n_dst; ++i) {
        if (!dsts[i]) return VAICU_ERR_INVALID_VALUE;
        if (reinterpret_cast<uintptr_t>(dsts[i]) & 15u) return VAICU_ERR_ALIGNMENT;
        spec.dst[i] = dsts[i];
    }
    return run_impl(pl, stream, I, W, nullptr, nullptr, dsts[0], workspace, &spec);
}

int vaicu_partial_fold_run(vaicu_device* dev, vaicu_stream_t stream, const void* parts, uint32_t n_parts, uint32_t rows, uint32_t N,
                           int part_dtype, const void* residual, float scale, int o_dtype, void* const* dsts, int n_dst, uint32_t row0)
{
    if (!dev || !parts || !dsts || n_parts == 0 || rows == 0 || N == 0 || n_dst < 1 || n_dst > 8) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(part_dtype) || !valid_dtype(o_dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)(row0 + rows) * N >= (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    if (reinterpret_cast<uintptr_t>(parts) & 15u) return VAICU_ERR_ALIGNMENT;
    for (int i = 0; i < n_dst; ++i) {
        if (!dsts[i]) return VAICU_ERR_INVALID_VALUE;
        if (reinterpret_cast<uintptr_t>(dsts[i]) & (dtype_size(o_dtype) - 1u)) return VAICU_ERR_ALIGNMENT;
    }
    if (residual && (reinterpret_cast<uintptr_t>(residual) & (dtype_size(o_dtype) - 1u))) return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_partial_fold(parts, n_parts, rows, N, part_dtype, residual, scale, o_dtype, dsts, (uint32_t)n_dst, row0,
                                   dev->sm_count, (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_peer_barrier_run(vaicu_device* dev, vaicu_stream_t stream, void* const* flag_arrays, int world, int rank, void* epoch_counter)
{
    if (!dev || !flag_arrays || !epoch_counter || world < 1 || world > 8 || rank < 0 || rank >= world) return VAICU_ERR_INVALID_VALUE;
    uint32_t* flags[8] = {};
    for (int i = 0; i < world; ++i) {
        if (!flag_arrays[i]) return VAICU_ERR_INVALID_VALUE;
        if (reinterpret_cast<uintptr_t>(flag_arrays[i]) & 3u) return VAICU_ERR_ALIGNMENT;
        flags[i] = reinterpret_cast<uint32_t*>(flag_arrays[i]);
    }
    if (reinterpret_cast<uintptr_t>(epoch_counter) & 3u) return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_peer_barrier(flags, world, rank, reinterpret_cast<uint32_t*>(epoch_counter), dev->status_word,
                                   (cudaStream_t)stream));
    return VAICU_OK;
}

namespace {
size_t argmax_ws_bytes(const vaicu_linear_plan* pl)
{
    if (pl->kernel != VAICU_KERNEL_GEMV || !pl->gemv_vec.vectorized || pl->d.gate_fuse) return 0;
    return 256u + align_up((size_t)pl->gemv_vec.grid * pl->d.M * 8u, 256u);
}
}  // namespace

int vaicu_linear_argmax_workspace_bytes(const vaicu_linear_plan* plan, size_t* out)
{
    if (!plan || !out) return VAICU_ERR_INVALID_VALUE;
    *out = argmax_ws_bytes(plan);
    return VAICU_OK;
}

int vaicu_linear_run_argmax(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W, const void* bias,
                            const void* residual, void* O, void* argmax_workspace, uint32_t index_base, float* out_val, void* out_u32)
{
    if (!pl || !I || !W || !argmax_workspace || !out_u32) return VAICU_ERR_INVALID_VALUE;
    const vaicu_linear_desc& d = pl->d;
    const size_t need = argmax_ws_bytes(pl);
    if (need == 0) return VAICU_ERR_UNSUPPORTED;             // not the weight-streaming kernel, or a gated Linear
    if (d.has_bias && !bias) return VAICU_ERR_INVALID_VALUE;
    if (d.has_residual && !residual) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)index_base + d.N > (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    auto elem_aligned = [](const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dtype_size(dt) - 1u)) == 0; };
    if (O && !elem_aligned(O, d.o_dtype)) return VAICU_ERR_ALIGNMENT;
    if (d.has_bias && !elem_aligned(bias, d.b_dtype)) return VAICU_ERR_ALIGNMENT;
    if (d.has_residual && !elem_aligned(residual, d.o_dtype)) return VAICU_ERR_ALIGNMENT;
    if ((reinterpret_cast<uintptr_t>(argmax_workspace) & 255u) || (reinterpret_cast<uintptr_t>(out_u32) & 3u) ||
        (reinterpret_cast<uintptr_t>(out_val) & 3u))
        return VAICU_ERR_ALIGNMENT;
    // the fused form exists for the 16-byte-vector kernel only; other views take the two-node path
    if (!aligned16(I) || !aligned16(W)) return VAICU_ERR_UNSUPPORTED;
    const LinearArgs a = make_args(d, I, W, d.has_bias ? bias : nullptr, d.has_residual ? residual : nullptr, O);
    uint8_t* ws = reinterpret_cast<uint8_t*>(argmax_workspace);
    GemvArgmax am{};
    am.count = reinterpret_cast<unsigned int*>(ws);
    am.block_val = reinterpret_cast<float*>(ws + 256u);
    am.block_idx = reinterpret_cast<uint32_t*>(am.block_val + (size_t)pl->gemv_vec.grid * d.M);
    am.out_val = out_val;
    am.out_idx = reinterpret_cast<uint32_t*>(out_u32);
    am.index_base = index_base;
    am.write_logits = O ? 1 : 0;
    pl->last_kernel = VAICU_KERNEL_GEMV;
    pl->last_vectorized = 1;
    VAICU_CUDA(launch_gemv(a, pl->gemv_vec, (cudaStream_t)stream, &am));
    return VAICU_OK;
}

int vaicu_linear_run_scatter(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W, const void* bias,
                             void* const* dsts, int n_dst, uint32_t ldo, uint32_t col0, void* workspace)
{
    if (!pl || !dsts || n_dst < 1 || n_dst > 8) return VAICU_ERR_INVALID_VALUE;
    const vaicu_linear_desc& d = pl->d;
    const uint32_t width = d.gate_fuse ? d.N / 2u : d.N;
    if (ldo < width || col0 > ldo - width) return VAICU_ERR_INVALID_VALUE;
    // only the tensor-core kernels write strided slabs, and only without a split-K fold or a residual
    if (!pl->tc || pl->tcp.splits > 1u || d.has_residual) return VAICU_ERR_UNSUPPORTED;
    OutputSpec spec{};
    spec.n_dst = (uint32_t)n_dst;
    spec.ldo = ldo;
    spec.col0 = col0;
    for (int i = 0; i < n_dst; ++i) {
        if (!dsts[i]) return VAICU_ERR_INVALID_VALUE;
        if (reinterpret_cast<uintptr_t>(dsts[i]) & 15u) return VAICU_ERR_ALIGNMENT;
        spec.dst[i] = dsts[i];
    }
    return run_impl(pl, stream, I, W, bias, nullptr, dsts[0], workspace, &spec);
}

int vaicu_linear_run_broadcast(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W, const void* bias,
                               const void* residual, void* const* dsts, int n_dst, void* workspace)
{
    if (!pl || !dsts || n_dst < 1 || n_dst > 8) return VAICU_ERR_INVALID_VALUE;
    const vaicu_linear_desc& d = pl->d;
    // the tensor-core kernels' epilogues store to several destinations; a split-K fold does not
    if (!pl->tc || pl->tcp.splits > 1u) return VAICU_ERR_UNSUPPORTED;
    OutputSpec spec{};
    spec.n_dst = (uint32_t)n_dst;
    spec.ldo = d.gate_fuse ? d.N / 2u : d.N;      // dense destinations: bias and residual index them like O
    spec.col0 = 0;
    for (int i = 0; i < n_dst; ++i) {
        if (!dsts[i]) return VAICU_ERR_INVALID_VALUE;
        if (reinterpret_cast<uintptr_t>(dsts[i]) & 15u) return VAICU_ERR_ALIGNMENT;
        spec.dst[i] = dsts[i];
    }
    return run_impl(pl, stream, I, W, bias, residual, dsts[0], workspace, &spec);
}

namespace {
int run_impl(vaicu_linear_plan* pl, vaicu_stream_t stream, const void* I, const void* W, const void* bias,
             const void* residual, void* O, void* workspace, const OutputSpec* spec)
{
    if (!pl || !I || !W || !O) return VAICU_ERR_INVALID_VALUE;
    const vaicu_linear_desc& d = pl->d;
    if (d.has_bias && !bias) return VAICU_ERR_INVALID_VALUE;
    if (d.has_residual && !residual) return VAICU_ERR_INVALID_VALUE;
    auto elem_aligned = [](const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dtype_size(dt) - 1u)) == 0; };
    if (!elem_aligned(I, d.i_dtype) || !elem_aligned(W, d.w_dtype) || !elem_aligned(O, d.o_dtype)) return VAICU_ERR_ALIGNMENT;
    if (d.has_bias && !elem_aligned(bias, d.b_dtype)) return VAICU_ERR_ALIGNMENT;
    if (d.has_residual && !elem_aligned(residual, d.o_dtype)) return VAICU_ERR_ALIGNMENT;
    if (pl->workspace_bytes && !workspace) return VAICU_ERR_WORKSPACE;
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u)) return VAICU_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const LinearArgs a = make_args(d, I, W, d.has_bias ? bias : nullptr, d.has_residual ? residual : nullptr, O);

    if (pl->kernel == VAICU_KERNEL_GEMV) {
        const bool vec = aligned16(I) && aligned16(W) && pl->gemv_vec.vectorized;
        pl->last_kernel = VAICU_KERNEL_GEMV;
        pl->last_vectorized = vec ? 1 : 0;
        VAICU_CUDA(launch_gemv(a, vec ? pl->gemv_vec : pl->gemv_any, s));
        return VAICU_OK;
    }
    pl->last_kernel = VAICU_KERNEL_FMA_TILE;
    pl->last_vectorized = 0;
    if (pl->kernel == VAICU_KERNEL_FMA_TILE) return run_fma(pl, a, workspace, s);

    // tensor-core path; operands TMA cannot address go to the FMA tile kernel
    if (!aligned16(W) || (!pl->tc_cast && !aligned16(I))) {
        if (spec) return VAICU_ERR_ALIGNMENT;      // the fallback kernel writes dense outputs only
        return run_fma(pl, a, workspace, s);
    }
    pl->last_kernel = pl->kernel;
    pl->last_vectorized = 1;
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    const void* act = I;
    if (pl->tc_cast) {
        VAICU_CUDA(launch_cast_f32_to_16(reinterpret_cast<const float*>(I), ws, d.w_dtype, (size_t)d.M * d.K, pl->dev->sm_count, s));
        act = ws;
    }
    float* partial = (pl->tcp.splits > 1u && !pl->tcp.cfold) ? reinterpret_cast<float*>(ws + pl->ws_cast_bytes) : nullptr;
    const bool gate = d.gate_fuse != 0;
    const void* a_base = pl->tc_swap ? W : act;
    const void* b_base = pl->tc_swap ? act : W;
    uint32_t ia = a_base == pl->map_a_base[0] ? 0u : (a_base == pl->map_a_base[1] ? 1u : 2u);
    if (ia == 2u) {                           // a base pointer not seen before: encode into the older slot
        ia = pl->map_a_next;
        pl->map_a_next ^= 1u;
        const uint32_t rows = pl->tc_swap ? d.N : d.M;
        int rc = encode_map(&pl->map_a[ia], a_base, d.w_dtype, rows, d.K, pl->tc_swap ? pl->tcp.tile_rows : 128u);
        if (rc != VAICU_OK) return rc;
        pl->map_a_base[ia] = a_base;
    }
    uint32_t ib = b_base == pl->map_b_base[0] ? 0u : (b_base == pl->map_b_base[1] ? 1u : 2u);
    if (ib == 2u) {
        ib = pl->map_b_next;
        pl->map_b_next ^= 1u;
        const uint32_t rows = pl->tc_swap ? d.M : d.N;
        const uint32_t box = ((gate && !pl->tc_swap) || pl->tcp.pair) ? pl->tcp.bn / 2u : pl->tcp.bn;
        int rc = encode_map(&pl->map_b[ib], b_base, d.w_dtype, rows, d.K, box);
        if (rc != VAICU_OK) return rc;
        pl->map_b_tail[ib] = pl->map_b[ib];
        if (pl->tcp.tail_split > 1u) {
            rc = encode_map(&pl->map_b_tail[ib], b_base, d.w_dtype, rows, d.K, pl->tcp.bn / pl->tcp.tail_split / 2u);
            if (rc != VAICU_OK) return rc;
        }
        pl->map_b_base[ib] = b_base;
    }
    TcParams t = pl->tcp;
    t.O = O; t.bias = a.bias; t.res = a.res; t.partial = partial;
    t.tile_done = partial ? pl->tile_done : nullptr;
    t.o_aligned16 = aligned16(O) ? 1u : 0u;
    t.n_dst = 1u;
    t.ldo = gate ? d.N / 2u : d.N;
    t.col0 = 0u;
    size_t smem = pl->tc_smem;
    if (spec) {
        t.n_dst = spec->n_dst; t.ldo = spec->ldo; t.col0 = spec->col0;
        for (uint32_t i = 0; i < spec->n_dst; ++i) t.dst[i] = spec->dst[i];
        t.rs_rows = spec->rs_rows;
        t.rs_slot = spec->rs_slot;
        if (t.pair && spec->n_dst > 1u) {
            // stores to peers go out as whole 128-byte row segments: one ring stage less, 16 KB of staging
            const uint32_t stage_bytes = 128u * 128u + (t.bn / 2u) * 128u;
            const uint32_t staged_stages = (uint32_t)((kTcMaxSmem - 2048u - 16384u - 128u) / stage_bytes);
            if (staged_stages >= 3u) {
                t.staged = 1u;
                t.stages = staged_stages < t.stages ? staged_stages : t.stages;
                smem = (size_t)t.stages * stage_bytes + 1024u + 256u + 16384u + 128u;
            }
        }
    }
    VAICU_CUDA(launch_tc_gemm(pl->map_a[ia], pl->map_b[ib], pl->map_b_tail[ib], t, pl->tc_swap, pl->tc_grid, smem, s));
    if (partial && !t.tile_done) VAICU_CUDA(launch_splitk_reduce(a, partial, t.splits, s));
    return VAICU_OK;
}
}  // namespace

int vaicu_ipc_export(const void* device_ptr, void* handle64)
{
    if (!device_ptr || !handle64) return VAICU_ERR_INVALID_VALUE;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    VAICU_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(device_ptr)));
    memcpy(handle64, &h, sizeof(h));
    return VAICU_OK;
}
int vaicu_ipc_open(const void* handle64, void** out_ptr)
{
    if (!handle64 || !out_ptr) return VAICU_ERR_INVALID_VALUE;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    VAICU_CUDA(cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return VAICU_OK;
}
int vaicu_ipc_close(void* ptr)
{
    if (!ptr) return VAICU_ERR_INVALID_VALUE;
    VAICU_CUDA(cudaIpcCloseMemHandle(ptr));
    return VAICU_OK;
}

namespace {
// Members of a group: one device and kernel family, one activation matrix, nothing after the dot product.
int group_members_ok(vaicu_linear_plan* const* plans, int count)
{
    if (!plans || count < 2 || count > 3 || !plans[0]) return VAICU_ERR_INVALID_VALUE;
    const vaicu_linear_plan* p0 = plans[0];
    uint64_t total = 0;
    for (int i = 0; i < count; ++i) {
        const vaicu_linear_plan* pl = plans[i];
        if (!pl) return VAICU_ERR_INVALID_VALUE;
        const vaicu_linear_desc& d = pl->d;
        const vaicu_linear_desc& d0 = p0->d;
        if (pl->dev != p0->dev || pl->kernel != p0->kernel) return VAICU_ERR_UNSUPPORTED;
        if (pl->kernel == VAICU_KERNEL_GEMV) {
            if (!pl->gemv_vec.vectorized) return VAICU_ERR_UNSUPPORTED;
        } else if (pl->kernel == VAICU_KERNEL_TC_SKINNY) {
            if (d.N % 128u) return VAICU_ERR_UNSUPPORTED;      // members are whole numbers of weight tiles
        } else if (pl->kernel == VAICU_KERNEL_TC_GEMM) {
            if (d.N % 256u || d.i_dtype == VAICU_DTYPE_F32) return VAICU_ERR_UNSUPPORTED;   // whole 256-column tiles, no cast pass
        } else {
            return VAICU_ERR_UNSUPPORTED;
        }
        if (d.M != d0.M || d.K != d0.K || d.i_dtype != d0.i_dtype || d.w_dtype != d0.w_dtype || d.o_dtype != d0.o_dtype)
            return VAICU_ERR_UNSUPPORTED;
        if (d.has_bias || d.has_residual || d.epilogue != VAICU_EPILOGUE_NONE || d.gate_fuse || d.scalar_scale != 1.0f)
            return VAICU_ERR_UNSUPPORTED;
        total += d.N;
    }
    if (total * p0->d.M >= (1ull << 32)) return VAICU_ERR_UNSUPPORTED;
    return VAICU_OK;
}

// The cached state of a tensor-core group, (re)built when the members change.
int group_state(vaicu_linear_plan* const* plans, int count, GroupState** out)
{
    vaicu_linear_plan* p0 = plans[0];
    GroupState* g = p0->group;
    bool same = g && g->count == count;
    // the same plans as last time, and still of the same sizes (a destroyed member's address may be reused)
    for (int i = 0; same && i < count; ++i) same = g->members[i] == plans[i] && g->rows[i] == plans[i]->d.N;
    if (!same) {
        if (g) { vaicu_linear_plan_destroy(g->virt); delete g; p0->group = nullptr; }
        g = new (std::nothrow) GroupState();
        if (!g) return VAICU_ERR_INVALID_VALUE;
        memset(g, 0, sizeof(*g));
        vaicu_linear_desc all = p0->d;
        uint32_t total = 0;
        for (int i = 0; i < count; ++i) { g->members[i] = plans[i]; g->rows[i] = plans[i]->d.N; total += plans[i]->d.N; }
        all.N = total;
        g->count = count;
        vaicu_linear_tuning tune = default_tuning();
        tune.kernel = p0->kernel;
        tune.tc_stages = p0->tune.tc_stages;
        if (p0->kernel == VAICU_KERNEL_TC_SKINNY) {
            tune.tc_splits = p0->tune.tc_splits;
            tune.tc_tile_rows = 128u;          // members begin at multiples of 128 rows
        } else {
            // CTA pairs, 256-column tiles (members are multiples of 256 columns), one K span, whole tiles only
            tune.tc_pair = 1;
            tune.tc_bn = 256u;
            tune.tc_splits = 1u;
            tune.tc_tail_strips = 1;
        }
        int rc = build_plan(p0->dev, &all, tune, &g->virt);
        if (rc == VAICU_OK && p0->kernel == VAICU_KERNEL_TC_GEMM && (!g->virt->tcp.pair || g->virt->tcp.splits != 1u)) {
            vaicu_linear_plan_destroy(g->virt);
            rc = VAICU_ERR_UNSUPPORTED;
        }
        if (rc != VAICU_OK) { delete g; return rc == VAICU_ERR_INVALID_VALUE ? VAICU_ERR_UNSUPPORTED : rc; }
        p0->group = g;
    }
    *out = g;
    return VAICU_OK;
}
}  // namespace

int vaicu_linear_group_workspace_bytes(vaicu_linear_plan* const* plans, int count, size_t* out_bytes)
{
    if (!out_bytes) return VAICU_ERR_INVALID_VALUE;
    int rc = group_members_ok(plans, count);
    if (rc != VAICU_OK) return rc;
    *out_bytes = 0;
    if (plans[0]->kernel == VAICU_KERNEL_GEMV) return VAICU_OK;
    GroupState* g = nullptr;
    rc = group_state(plans, count, &g);
    if (rc != VAICU_OK) return rc;
    const vaicu_linear_plan* v = g->virt;
    if (plans[0]->kernel == VAICU_KERNEL_TC_GEMM) return VAICU_OK;      // the members' outputs leave through the epilogue
    *out_bytes = v->ws_cast_bytes + (v->tcp.cfold ? 0u : align_up((size_t)v->tcp.splits * v->d.M * v->d.N * sizeof(float), 256u));
    return VAICU_OK;
}

int vaicu_linear_run_group(vaicu_linear_plan* const* plans, int count, vaicu_stream_t stream, const void* I,
                           const void* const* W, void* const* O, void* workspace)
{
    if (!W || !O || !I) return VAICU_ERR_INVALID_VALUE;
    int rc = group_members_ok(plans, count);
    if (rc != VAICU_OK) return rc;
    vaicu_linear_plan* p0 = plans[0];
    uint32_t rows[3] = {0, 0, 0};
    uint64_t total = 0;
    for (int i = 0; i < count; ++i) {
        if (!W[i] || !O[i]) return VAICU_ERR_INVALID_VALUE;
        if (!aligned16(W[i])) return VAICU_ERR_UNSUPPORTED;
        rows[i] = plans[i]->d.N;
        total += rows[i];
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (p0->kernel == VAICU_KERNEL_GEMV) {
        if (!aligned16(I)) return VAICU_ERR_UNSUPPORTED;
        vaicu_linear_desc all = p0->d;
        all.N = (uint32_t)total;
        LinearArgs a = make_args(all, I, W[0], nullptr, nullptr, O[0]);
        const GemvConfig cfg = choose_gemv(a, p0->dev->sm_count, true, &p0->tune);
        if (!cfg.vectorized) return VAICU_ERR_UNSUPPORTED;
        VAICU_CUDA(launch_gemv_group(a, cfg, (uint32_t)count, rows, W, O, s));
        return VAICU_OK;
    }
    // swapped tensor-core kernel: one launch leaves the partial sums of all members, one fold stores the outputs
    for (int i = 0; i < count; ++i)
        if (!aligned16(O[i])) return VAICU_ERR_UNSUPPORTED;
    GroupState* g = nullptr;
    rc = group_state(plans, count, &g);
    if (rc != VAICU_OK) return rc;
    vaicu_linear_plan* v = g->virt;
    const vaicu_linear_desc& d = v->d;
    if (p0->kernel == VAICU_KERNEL_TC_GEMM) {
        // CTA-pair kernel: one GEMM over the members' weight rows side by side (9 rounds of tiles for the q / k / v
        // of a 3B-class model at M = 8192 where three launches take 6 + 2 + 2), each tile stored to its member
        if (!aligned16(I)) return VAICU_ERR_UNSUPPORTED;
        for (int i = 0; i < count; ++i) {
            if (g->w_base[i] == W[i]) continue;
            rc = encode_map(&g->maps_w[i], W[i], d.w_dtype, rows[i], d.K, 128u);      // each CTA of a pair stages 128 of the 256 rows
            if (rc != VAICU_OK) return rc;
            g->w_base[i] = W[i];
        }
        if (count == 2) g->maps_w[2] = g->maps_w[1];
        uint32_t ia = I == g->act_base[0] ? 0u : (I == g->act_base[1] ? 1u : 2u);
        if (ia == 2u) {
            ia = g->act_next;
            g->act_next ^= 1u;
            rc = encode_map(&g->map_act[ia], I, d.w_dtype, d.M, d.K, 128u);
            if (rc != VAICU_OK) return rc;
            g->act_base[ia] = I;
        }
        TcParams t = v->tcp;
        t.O = nullptr; t.bias = nullptr; t.res = nullptr; t.partial = nullptr; t.tile_done = nullptr;
        t.n_dst = 1u; t.ldo = d.N; t.col0 = 0u; t.o_aligned16 = 1u;
        t.grp_t1 = rows[0] / 256u;
        t.grp_t2 = count > 2 ? (rows[0] + rows[1]) / 256u : kNoGroup;
        for (int i = 0; i < count; ++i) t.dst[i] = O[i];
        VAICU_CUDA(launch_tc_pair_group(g->map_act[ia], g->maps_w, t, v->tc_grid, v->tc_smem, s));
        for (int i = 0; i < count; ++i) { plans[i]->last_kernel = VAICU_KERNEL_TC_GEMM; plans[i]->last_vectorized = 1; }
        return VAICU_OK;
    }
    if (!v->tc_cast && !aligned16(I)) return VAICU_ERR_UNSUPPORTED;
    if (v->tc_cast && (reinterpret_cast<uintptr_t>(I) & 3u)) return VAICU_ERR_ALIGNMENT;
    const bool in_cluster = v->tcp.cfold != 0u;       // the K splits fold inside clusters: no partial sums, no fold launch
    if (!workspace && (v->tc_cast || !in_cluster)) return VAICU_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return VAICU_ERR_ALIGNMENT;
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    const void* act = I;
    if (v->tc_cast) {
        VAICU_CUDA(launch_cast_f32_to_16(reinterpret_cast<const float*>(I), ws, d.w_dtype, (size_t)d.M * d.K, p0->dev->sm_count, s));
        act = ws;
    }
    float* partial = reinterpret_cast<float*>(ws + v->ws_cast_bytes);
    for (int i = 0; i < count; ++i) {
        if (g->w_base[i] == W[i]) continue;
        rc = encode_map(&g->maps_w[i], W[i], d.w_dtype, rows[i], d.K, 128u);
        if (rc != VAICU_OK) return rc;
        g->w_base[i] = W[i];
    }
    if (count == 2) g->maps_w[2] = g->maps_w[1];
    uint32_t ib = act == g->act_base[0] ? 0u : (act == g->act_base[1] ? 1u : 2u);
    if (ib == 2u) {
        ib = g->act_next;
        g->act_next ^= 1u;
        rc = encode_map(&g->map_act[ib], act, d.w_dtype, d.M, d.K, v->tcp.bn);
        if (rc != VAICU_OK) return rc;
        g->act_base[ib] = act;
    }
    TcParams t = v->tcp;
    t.O = nullptr; t.bias = nullptr; t.res = nullptr; t.partial = in_cluster ? nullptr : partial; t.tile_done = nullptr;
    t.n_dst = 1u; t.ldo = d.N; t.col0 = 0u;
    t.grp_t1 = rows[0] / 128u;
    t.grp_t2 = count > 2 ? (rows[0] + rows[1]) / 128u : kNoGroup;
    for (int i = 0; i < count; ++i) t.dst[i] = O[i];
    VAICU_CUDA(launch_tc_gemm_group(g->maps_w, g->map_act[ib], t, v->tc_grid, v->tc_smem, s));
    if (!in_cluster) VAICU_CUDA(launch_group_fold(partial, t.splits, d.M, (uint32_t)count, rows, O, d.o_dtype, s));
    for (int i = 0; i < count; ++i) { plans[i]->last_kernel = VAICU_KERNEL_TC_SKINNY; plans[i]->last_vectorized = 1; }
    return VAICU_OK;
}

int vaicu_rms_norm_run(vaicu_device* dev, vaicu_stream_t stream, const void* in, const void* scale, const void* shift,
                       const void* residual, void* out, uint32_t rows, uint32_t feat, int i_dtype, int w_dtype, int o_dtype,
                       float eps)
{
    if (!dev || !in || !out || rows == 0 || feat == 0) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(i_dtype) || !valid_dtype(o_dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((scale || shift) && !valid_dtype(w_dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)rows * feat >= (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(in) & (dtype_size(i_dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out) & (dtype_size(o_dtype) - 1u)))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_rms_norm(in, scale, shift, residual, out, rows, feat, i_dtype, w_dtype, o_dtype, eps, dev->sm_count,
                               (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_layer_norm_run(vaicu_device* dev, vaicu_stream_t stream, const void* in, const void* scale, const void* shift,
                       const void* residual, void* out, uint32_t rows, uint32_t feat, int i_dtype, int w_dtype, int o_dtype,
                       float eps)
{
    if (!dev || !in || !out || !scale || rows == 0 || feat == 0) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(i_dtype) || !valid_dtype(o_dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((scale || shift) && !valid_dtype(w_dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)rows * feat >= (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(in) & (dtype_size(i_dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out) & (dtype_size(o_dtype) - 1u)))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_layer_norm(in, scale, shift, residual, out, rows, feat, i_dtype, w_dtype, o_dtype, eps, dev->sm_count,
                               (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_gated_mul_run(vaicu_device* dev, vaicu_stream_t stream, const void* in, void* out, uint32_t rows, uint32_t H,
                        int i_dtype, int o_dtype, int activation)
{
    if (!dev || !in || !out || rows == 0 || H == 0) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(i_dtype) || !valid_dtype(o_dtype)) return VAICU_ERR_INVALID_VALUE;
    if (activation < 0 || activation > VAICU_EPILOGUE_SIGMOID) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)rows * H * 2u >= (1ull << 32)) return VAICU_ERR_INVALID_VALUE;      // vAi indexes with uint32
    if ((reinterpret_cast<uintptr_t>(in) & (dtype_size(i_dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out) & (dtype_size(o_dtype) - 1u)))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_gated_mul(in, out, rows, H, i_dtype, o_dtype, activation, dev->sm_count, (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_argmax_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, void* out_u32)
{
    if (!logits || !out_u32 || M == 0 || N == 0) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(logits) & (dtype_size(dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out_u32) & 3u))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_argmax(logits, dtype, M, N, reinterpret_cast<uint32_t*>(out_u32), (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_argmax_workspace_bytes(uint32_t M, uint32_t N, size_t* out_bytes)
{
    if (!out_bytes || M == 0 || N == 0) return VAICU_ERR_INVALID_VALUE;
    *out_bytes = align_up((size_t)M * argmax_parts(N) * 8u, 256u);
    return VAICU_OK;
}

int vaicu_argmax_pairs_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, size_t ld,
                           uint32_t index_base, void* workspace, float* out_val, void* out_u32)
{
    if (!logits || !out_u32 || !workspace || M == 0 || N == 0 || ld < N) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)index_base + N > (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(logits) & (dtype_size(dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out_u32) & 3u) ||
        (reinterpret_cast<uintptr_t>(out_val) & 3u) || (reinterpret_cast<uintptr_t>(workspace) & 15u))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_argmax_pairs(logits, dtype, M, N, ld, index_base, workspace, out_val, reinterpret_cast<uint32_t*>(out_u32),
                                   (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_argmax_merge_run(vaicu_stream_t stream, const float* vals, const void* idx_u32, uint32_t groups, size_t group_stride,
                           uint32_t M, float* out_val, void* out_u32)
{
    if (!vals || !idx_u32 || !out_u32 || groups == 0 || M == 0 || group_stride < M) return VAICU_ERR_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(vals) & 3u) || (reinterpret_cast<uintptr_t>(idx_u32) & 3u) ||
        (reinterpret_cast<uintptr_t>(out_u32) & 3u) || (reinterpret_cast<uintptr_t>(out_val) & 3u))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_argmax_merge(vals, reinterpret_cast<const uint32_t*>(idx_u32), groups, group_stride, M, out_val,
                                   reinterpret_cast<uint32_t*>(out_u32), (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_topk_workspace_bytes(uint32_t M, uint32_t N, uint32_t k, size_t* out_bytes)
{
    if (!out_bytes || M == 0 || N == 0 || k == 0 || k > 128u) return VAICU_ERR_INVALID_VALUE;
    const uint32_t G = topk_groups(N);
    *out_bytes = G == 1u ? 0 : align_up((size_t)M * G * (k < N ? k : N) * 8u, 256u);
    return VAICU_OK;
}

int vaicu_topk_sample_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, uint32_t k,
                          float temperature, const float* u_device, void* workspace, void* out_u32)
{
    if (!logits || !out_u32 || !u_device || M == 0 || N == 0 || k == 0 || k > 128u) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(dtype)) return VAICU_ERR_INVALID_VALUE;
    const uint32_t G = topk_groups(N);
    if (G > 1u && !workspace) return VAICU_ERR_WORKSPACE;
    // stage 2 walks the G slice lists with one warp, at most 8 per lane
    if (G > 256u) return VAICU_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(logits) & (dtype_size(dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out_u32) & 3u) ||
        (reinterpret_cast<uintptr_t>(u_device) & 3u) || (reinterpret_cast<uintptr_t>(workspace) & 7u))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_topk_sample(logits, dtype, M, N, k, temperature, u_device, workspace, reinterpret_cast<uint32_t*>(out_u32),
                                  (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_topk_candidates_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, size_t ld, uint32_t k,
                              uint32_t index_base, void* workspace, void* out_pairs)
{
    if (!logits || !out_pairs || M == 0 || N == 0 || k == 0 || k > 128u || ld < N) return VAICU_ERR_INVALID_VALUE;
    if (!valid_dtype(dtype)) return VAICU_ERR_INVALID_VALUE;
    if ((uint64_t)index_base + N > (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    const uint32_t G = topk_groups(N);
    if (G > 1u && !workspace) return VAICU_ERR_WORKSPACE;
    if (G > 256u) return VAICU_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(logits) & (dtype_size(dtype) - 1u)) || (reinterpret_cast<uintptr_t>(out_pairs) & 7u) ||
        (reinterpret_cast<uintptr_t>(workspace) & 7u))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_topk(logits, dtype, M, N, ld, k, index_base, 1.0f, nullptr, workspace, nullptr, out_pairs, (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_topk_merge_sample_run(vaicu_stream_t stream, const void* pairs, uint32_t groups, size_t group_stride, uint32_t M,
                                uint32_t list_len, uint32_t k, float temperature, const float* u_device, void* out_u32)
{
    if (!pairs || !u_device || !out_u32 || groups == 0 || groups > 256u || M == 0 || list_len == 0 || k == 0 || k > 128u)
        return VAICU_ERR_INVALID_VALUE;
    if (k > list_len * groups || group_stride < (size_t)M * list_len) return VAICU_ERR_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(pairs) & 7u) || (reinterpret_cast<uintptr_t>(u_device) & 3u) || (reinterpret_cast<uintptr_t>(out_u32) & 3u))
        return VAICU_ERR_ALIGNMENT;
    VAICU_CUDA(launch_topk_merge_sample(pairs, groups, group_stride, M, list_len, k, temperature, u_device,
                                        reinterpret_cast<uint32_t*>(out_u32), (cudaStream_t)stream));
    return VAICU_OK;
}

int vaicu_linear_shard_desc(const vaicu_linear_desc* full, int rank, int world, vaicu_linear_desc* shard,
                            uint32_t* w_row_begin, uint32_t* w_row_count)
{
    if (!full || !shard || !w_row_begin || !w_row_count || world <= 0 || rank < 0 || rank >= world) return VAICU_ERR_INVALID_VALUE;
    const uint32_t H = full->gate_fuse ? full->N / 2u : full->N;
    if (full->gate_fuse && full->N % 2u) return VAICU_ERR_INVALID_VALUE;
    // a column split keeps only per-column operands local; anything indexed over the whole of O is not sharded here
    if (full->has_residual) return VAICU_ERR_UNSUPPORTED;
    if (full->has_bias && full->bias_elems != full->N && !(full->bias_elems == 0 && full->M == 1u))
        return VAICU_ERR_UNSUPPORTED;
    const uint32_t base = H / (uint32_t)world, extra = H % (uint32_t)world;
    const uint32_t begin = (uint32_t)rank * base + ((uint32_t)rank < extra ? (uint32_t)rank : extra);
    const uint32_t count = base + ((uint32_t)rank < extra ? 1u : 0u);
    if (count == 0) return VAICU_ERR_INVALID_VALUE;
    *shard = *full;
    shard->N = full->gate_fuse ? 2u * count : count;
    if (full->has_bias) shard->bias_elems = shard->N;
    *w_row_begin = begin;
    *w_row_count = count;
    return VAICU_OK;
}

const char* vaicu_status_string(int status)
{
    switch (status) {
    case VAICU_OK: return "ok";
    case VAICU_ERR_INVALID_VALUE: return "invalid value (null pointer, bad enum or shape)";
    case VAICU_ERR_UNSUPPORTED: return "unsupported combination";
    case VAICU_ERR_CUDA: return "CUDA call failed";
    case VAICU_ERR_NO_DEVICE: return "no usable sm_100 device or driver";
    case VAICU_ERR_WORKSPACE: return "workspace missing or too small";
    case VAICU_ERR_ALIGNMENT: return "pointer alignment";
    case VAICU_ERR_TOO_LARGE: return "shape exceeds the fixed capacity of this entry point";
    case VAICU_ERR_TIMEOUT: return "a bounded device-side wait expired";
    default: return "unknown status";
    }
}
const char* vaicu_last_cuda_error(void) { return g_last_error; }
int vaicu_version(void) { return 1000; }

}  // extern "C"
#pragma GCC visibility pop
