// Decode path of Linear: M <= 8 rows of activations against W [N, K].
//
// Stands where vAi's slab kernel does (vai/shaders/linear-slab.comp, chosen by
// Linear::useSlabPath, vai/nodes/linear.h:320): one pass over the weights, fp32
// accumulation, bias / epilogue / residual / scale fused into the store.  The
// design is for HBM bandwidth on B200 rather than a translation of that shader:
//   * every lane streams 16-byte weight vectors with ld.global.nc (no L1
//     allocation); a warp reads 512 contiguous bytes of each of its R rows per
//     step and keeps 2*R such loads in flight;
//   * the activations are converted to fp32 once per block and kept in shared
//     memory, laid out so that the float4 reads are bank-conflict free;
//   * K is split over `k_warps` warps of a block when N alone cannot fill
//     148 SMs; the fold goes through shared memory, no global scratch;
//   * blocks are persistent over row groups (grid sized to the SM count).
#include "common.cuh"

namespace vaicu {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// A 16-byte weight vector as packed float2 pairs (element 2i, element 2i+1).
template <typename TW> struct WTraits;
template <> struct WTraits<float> {
    static constexpr int VEC = 4;
    __device__ static __forceinline__ void unpack(const uint4& v, float2* f)
    {
        f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
        f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
    }
};
template <> struct WTraits<__half> {
    static constexpr int VEC = 8;
    __device__ static __forceinline__ void unpack(const uint4& v, float2* f)
    {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
};
template <> struct WTraits<__nv_bfloat16> {
    static constexpr int VEC = 8;
    __device__ static __forceinline__ void unpack(const uint4& v, float2* f)
    {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
    }
};

__device__ __forceinline__ uint4 ldg_stream(const void* p)
{
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Position of chunk-relative element kk inside the staged activations.  With
// 8-element weight vectors a lane needs two float4 per step; splitting every
// 256-element segment into two 128-float planes keeps both reads conflict free.
template <int VEC> __device__ __forceinline__ uint32_t xs_pos(uint32_t kk)
{
    if (VEC == 4) return kk;
    const uint32_t seg = kk & ~255u, r = kk & 255u;
    return seg + ((r & 4u) << 5) + ((r >> 3) << 2) + (r & 3u);
}

struct GemvParams {
    LinearArgs a;
    uint32_t H;          // output columns (N, or N/2 when gate_fuse)
    uint32_t cols_per_warp;
    uint32_t k_warps;    // warps splitting K inside a block
    uint32_t k_chunk;    // activations staged per round (multiple of 256)
    uint32_t k_pad;      // floats reserved per activation row in shared memory
    // Grouped launch (nseg > 0): up to 3 plain Linears that share the activations run
    // as one kernel over the concatenation of their weight rows.
    uint32_t nseg;
    uint32_t seg_begin[4];   // first virtual row of each segment; [nseg] = total rows
    const void* seg_w[3];
    void* seg_o[3];
    // Argmax folded into the launch (am.out_idx != null): plain Linears only, no gate, no group.
    GemvArgmax am;
#ifdef VAICU_GEMV_TRACE
    uint32_t trace_id;   // which launch of the recorded chain this is
#endif
};

// Four consecutive activations (chunk-relative kk, kk % 4 == 0) of row m -> fp32 in
// shared memory.  K % 4 == 0 and a 16-byte aligned base make every load aligned.
template <int VEC>
__device__ __forceinline__ void stage4(const LinearArgs& a, float* xs_row, uint32_t m, uint32_t c0, uint32_t kk)
{
    const size_t g = (size_t)m * a.K + c0 + kk;
    float4 v;
    if (a.i_dtype == VAICU_DTYPE_F32) {
        v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.I) + g);
    } else {
        const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.I) + g);
        if (a.i_dtype == VAICU_DTYPE_F16) {
            const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
            const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
            v = make_float4(p0.x, p0.y, p1.x, p1.y);
        } else {
            v = make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xFFFF0000u),
                            __uint_as_float(w.y << 16), __uint_as_float(w.y & 0xFFFF0000u));
        }
    }
    *reinterpret_cast<float4*>(xs_row + xs_pos<VEC>(kk)) = v;
}

// VEC consecutive activations of row 0 straight from global memory as float2 pairs
// (M = 1 only: with a single activation row there is nothing to share through shared
// memory, and skipping the staging round removes a barrier from every short kernel).
template <int VEC>
__device__ __forceinline__ void load_x_direct(const LinearArgs& a, uint32_t k, float2* xf)
{
    if (a.i_dtype == VAICU_DTYPE_F32) {
        const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.I) + k);
        const float4 t0 = s[0];
        xf[0] = make_float2(t0.x, t0.y); xf[1] = make_float2(t0.z, t0.w);
        if (VEC == 8) {
            const float4 t1 = s[1];
            xf[2 % (VEC / 2)] = make_float2(t1.x, t1.y); xf[3 % (VEC / 2)] = make_float2(t1.z, t1.w);
        }
    } else {
        uint32_t w[4];
        const uint16_t* s = reinterpret_cast<const uint16_t*>(a.I) + k;
        if (VEC == 8) {
            const uint4 t = *reinterpret_cast<const uint4*>(s);
            w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
        } else {
            const uint2 t = *reinterpret_cast<const uint2*>(s);
            w[0] = t.x; w[1] = t.y; w[2] = 0; w[3] = 0;
        }
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i)
            xf[i] = a.i_dtype == VAICU_DTYPE_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&w[i]))
                                                 : make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
    }
}

// R rows of W per warp step.  With gate_fuse the R rows are R/2 gate rows and
// the R/2 value rows of the same output columns.  Sums are kept as float2 pairs
// (even / odd elements) and advanced with the packed fp32 FMA of sm_100, which
// halves the FMA issue count: the kernel must stay memory-bound up to M = 8.
#ifdef VAICU_GEMV_TRACE
// Development aid (not built by default): phase time stamps of every block of every launch of a recorded chain.
__device__ unsigned long long g_gemv_trace[96 * 512 * 6];
static unsigned g_gemv_trace_next = 0;
__device__ __forceinline__ void gemv_trace(uint32_t launch, uint32_t slot)
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (launch < 96u && blockIdx.x < 512u) g_gemv_trace[((size_t)launch * 512u + blockIdx.x) * 6u + slot] = t;
}
#define GEMV_TRACE(slot) do { if (threadIdx.x == 0) gemv_trace(p.trace_id, slot); } while (0)
#else
#define GEMV_TRACE(slot)
#endif

template <typename TW, int M, int R, int U>
__global__ void __launch_bounds__(kThreads, (M == 1 && R * U <= 8) ? 3 : 2) gemv_kernel(const GemvParams p)
{
    constexpr int VEC = WTraits<TW>::VEC;
    constexpr int PAIRS = VEC / 2;
    constexpr bool DIRECT = (M == 1);     // activations read from global memory, not staged
    extern __shared__ __align__(16) float smem_f[];
    float* xs = smem_f;                               // [M][k_pad]
    float* red = smem_f + (size_t)M * p.k_pad;        // [kWarps][R*M]

    launch_dependents();
    GEMV_TRACE(0);

    const LinearArgs& a = p.a;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t KS = p.k_warps, RG = kWarps / KS;
    const uint32_t rg = warp / KS, ks = warp % KS;
    const uint32_t K = a.K, H = p.H;
    const bool gate = a.gate_fuse != 0;
    const uint32_t C = p.cols_per_warp;               // R, or R/2 with gate
    const uint32_t ngroups = (H + C - 1u) / C;
    const uint32_t nblocks = (ngroups + RG - 1u) / RG;
    const uint32_t stride = KS * 32u * VEC;
    const uint32_t nchunks = (K + p.k_chunk - 1u) / p.k_chunk;
    const EpilogueArgs ep = make_epilogue_args(a);
    const TW* Wp = reinterpret_cast<const TW*>(a.W);
    const uint32_t kk0 = (ks * 32u + lane) * VEC;
    bool staged = false;
    uint4 wv[U][R];           // one trip of weights: U k-steps of R rows per lane
    bool preloaded = false;   // wv already holds the first trip (loaded ahead of the dependency wait)
    const bool with_argmax = p.am.out_idx != nullptr;
    float am_best = kArgmaxLowest;          // this lane's best output so far (its batch row m = lane % M)
    uint32_t am_at = 0xFFFFFFFFu;

    // Row pointers of the R rows this warp takes in block-task pb.
    const TW* rowp[R];
    auto set_rows = [&](uint32_t pb) {
        const uint32_t j0 = (pb * RG + rg) * C;       // may be past the last group: rows clamp, stores skip
#pragma unroll
        for (int r = 0; r < R; ++r) {
            uint32_t row;
            if (gate) row = (r < R / 2) ? (j0 + r) : (H + j0 + (r - R / 2));
            else row = j0 + r;
            const uint32_t lim = gate ? ((r < R / 2) ? H - 1u : 2u * H - 1u) : (a.N - 1u);
            row = row < lim ? row : lim;
            if (p.nseg) {
                const uint32_t sg = (row >= p.seg_begin[1] ? 1u : 0u) + (row >= p.seg_begin[2] ? 1u : 0u);
                rowp[r] = reinterpret_cast<const TW*>(p.seg_w[sg]) + (size_t)(row - p.seg_begin[sg]) * K;
            } else {
                rowp[r] = Wp + (size_t)row * K;
            }
        }
    };
    // The first trip of a task's weights (first activation chunk) into registers.
    const uint32_t first_span = p.k_chunk < K ? p.k_chunk : K;
    auto preload = [&]() {
        const uint32_t iters0 = (first_span + stride - 1u) / stride;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t kk = kk0 + (uint32_t)u * stride;
            const bool v = ((uint32_t)u < iters0) && (kk < first_span);
#pragma unroll
            for (int r = 0; r < R; ++r) wv[u][r] = v ? ldg_stream(rowp[r] + kk) : make_uint4(0, 0, 0, 0);
        }
    };
    if (blockIdx.x < nblocks) set_rows(blockIdx.x);

    for (uint32_t pb = blockIdx.x; pb < nblocks; pb += gridDim.x) {
        const uint32_t g = pb * RG + rg;              // may be >= ngroups: rows clamp, stores skip
        const uint32_t j0 = g * C;
        if (!staged) {
            // The weights do not depend on the previous kernel: pull this warp's first
            // vectors toward L2 while that kernel drains, then wait for its results.
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (uint32_t it = 0; it < 8u; ++it)
                    if (kk0 + it * stride < first_span) prefetch_l2(rowp[r] + kk0 + it * stride);
            // ... and this warp's first trip goes all the way into registers: its loads are
            // in flight while the wait below and the activation staging run
            preload();
            preloaded = true;
            GEMV_TRACE(1);
            dependency_wait();
            GEMV_TRACE(2);
            if (DIRECT) staged = true;
        }
        // Bias and residual of the output this lane will store, requested ahead of the dot product
        // (the residual may come from the launch ahead: after the wait above).
        float early_bias = 0.0f, early_res = 0.0f;
        if (!gate && !p.nseg && ks == 0u && g < ngroups && lane < (uint32_t)(R * M)) {
            const uint32_t n = j0 + lane / M;
            if (n < a.N) {
                const size_t flat = (size_t)(lane % M) * a.N + n;
                early_bias = read_bias(ep, flat);
                early_res = read_res(ep, flat);
            }
        }
        float2 acc[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = make_float2(0.0f, 0.0f);

        for (uint32_t ch = 0; ch < nchunks; ++ch) {
            const uint32_t c0 = ch * p.k_chunk;
            const uint32_t c1 = (c0 + p.k_chunk < K) ? c0 + p.k_chunk : K;
            const uint32_t span = c1 - c0;
            if (!DIRECT && (nchunks > 1u || !staged)) {
                if (staged) __syncthreads();
                const uint32_t quads = span >> 2;
                for (uint32_t i = threadIdx.x; i < (uint32_t)M * quads; i += kThreads) {
                    const uint32_t m = (M == 1) ? 0u : i / quads;
                    const uint32_t kk = (i - m * quads) << 2;
                    stage4<VEC>(a, xs + (size_t)m * p.k_pad, m, c0, kk);
                }
                __syncthreads();
                staged = true;
            }
            const uint32_t iters = (span + stride - 1u) / stride;
            for (uint32_t it = 0; it < iters; it += U) {
                // U k-steps of R rows: U * R 16-byte loads in flight per lane
                bool valid[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t kk = kk0 + (it + u) * stride;
                    valid[u] = (it + u < iters) && (kk < span);
                }
                if (!preloaded) {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const uint32_t kk = kk0 + (it + u) * stride;
#pragma unroll
                        for (int r = 0; r < R; ++r)
                            wv[u][r] = valid[u] ? ldg_stream(rowp[r] + c0 + kk) : make_uint4(0, 0, 0, 0);
                    }
                }
                preloaded = false;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (!valid[u]) continue;
                    const uint32_t kk = kk0 + (it + u) * stride;
                    float2 xf[M][PAIRS];
                    if (DIRECT) load_x_direct<VEC>(a, c0 + kk, xf[0]);
#pragma unroll
                    for (int m = 0; m < (DIRECT ? 0 : M); ++m) {
                        const float* xrow = xs + (size_t)m * p.k_pad;
                        if (VEC == 4) {
                            const float4 t = *reinterpret_cast<const float4*>(xrow + kk);
                            xf[m][0] = make_float2(t.x, t.y); xf[m][1] = make_float2(t.z, t.w);
                        } else {
                            const uint32_t base = (kk & ~255u) + ((kk & 255u) >> 1);   // lane*4 within the segment
                            const float4 t0 = *reinterpret_cast<const float4*>(xrow + base);
                            const float4 t1 = *reinterpret_cast<const float4*>(xrow + base + 128);
                            xf[m][0] = make_float2(t0.x, t0.y); xf[m][1] = make_float2(t0.z, t0.w);
                            xf[m][2 % PAIRS] = make_float2(t1.x, t1.y); xf[m][3 % PAIRS] = make_float2(t1.z, t1.w);
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        float2 wf[PAIRS];
                        WTraits<TW>::unpack(wv[u][r], wf);
#pragma unroll
                        for (int m = 0; m < M; ++m)
#pragma unroll
                            for (int e = 0; e < PAIRS; ++e) acc[r][m] = __ffma2_rn(wf[e], xf[m][e], acc[r][m]);
                    }
                }
            }
        }

        if (pb == blockIdx.x) GEMV_TRACE(3);
        // The next task's first trip is requested now, so that it is in flight while this task's sums
        // are folded and stored (the registers of this task's last trip are free).
        if (pb + gridDim.x < nblocks) {
            set_rows(pb + gridDim.x);
            preload();
            preloaded = true;
        }
        // fold the pair and the 32 lanes of each warp
        float sums[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float v = acc[r][m].x + acc[r][m].y;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                sums[r][m] = v;
            }
        // this lane's (row r, batch m) pair
        float mine = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (lane == (uint32_t)(r * M + m)) mine = sums[r][m];
        if (KS > 1u) {
            if (lane < (uint32_t)(R * M)) red[warp * (R * M) + lane] = mine;
            __syncthreads();
            if (ks == 0u && lane < (uint32_t)(R * M)) {
                mine = 0.0f;
                for (uint32_t s = 0; s < KS; ++s) mine += red[(rg * KS + s) * (R * M) + lane];
            }
        }
        if (ks == 0u && g < ngroups) {
            if (!gate) {
                if (lane < (uint32_t)(R * M)) {
                    const uint32_t r = lane / M, m = lane % M;
                    const uint32_t n = j0 + r;
                    if (n < a.N) {
                        if (p.nseg) {
                            const uint32_t sg = (n >= p.seg_begin[1] ? 1u : 0u) + (n >= p.seg_begin[2] ? 1u : 0u);
                            const uint32_t width = p.seg_begin[sg + 1] - p.seg_begin[sg];
                            store_from_f32(p.seg_o[sg], a.o_dtype, (size_t)m * width + (n - p.seg_begin[sg]), mine);
                        } else {
                            const size_t flat = (size_t)m * a.N + n;
                            const float v = finish_output_pre(ep, mine, early_bias, early_res);
                            if (!with_argmax || p.am.write_logits) store_from_f32(a.O, a.o_dtype, flat, v);
                            // the Argmax node reads the stored logits: compare what the store would hold
                            if (with_argmax) argmax_take(round_through(a.o_dtype, v), p.am.index_base + n, am_best, am_at);
                        }
                    }
                }
            } else {
                // rows r < R/2 hold gate sums, rows r + R/2 the value sums of the same column
                const float up = __shfl_sync(0xFFFFFFFFu, mine, (lane + (R / 2) * M) & 31u);
                if (lane < (uint32_t)((R / 2) * M)) {
                    const uint32_t r = lane / M, m = lane % M;
                    const uint32_t j = j0 + r;
                    if (j < H) {
                        const size_t flat = (size_t)m * H + j;
                        store_from_f32(a.O, a.o_dtype, flat, finish_gated(ep, mine, up, j, H, flat));
                    }
                }
            }
        }
        if (KS > 1u) __syncthreads();   // red is reused by the next row group
    }
    GEMV_TRACE(4);

    if (with_argmax) {
        // 1. the block's candidate per batch row: lanes r * M + m of the store warps hold results
        __shared__ float s_val[kThreads];
        __shared__ uint32_t s_at[kThreads];
        __shared__ bool s_last;
        s_val[threadIdx.x] = am_best;
        s_at[threadIdx.x] = am_at;
        __syncthreads();
        if (threadIdx.x < (uint32_t)M) {
            float best = kArgmaxLowest;
            uint32_t at = 0xFFFFFFFFu;
            for (uint32_t w = 0; w < (uint32_t)kWarps; ++w)
#pragma unroll
                for (int r = 0; r < R; ++r) argmax_take(s_val[w * 32u + r * M + threadIdx.x], s_at[w * 32u + r * M + threadIdx.x], best, at);
            p.am.block_val[(size_t)blockIdx.x * M + threadIdx.x] = best;
            p.am.block_idx[(size_t)blockIdx.x * M + threadIdx.x] = at;
            __threadfence();                           // candidates visible before the ticket below
        }
        __syncthreads();
        // 2. the last block to take a ticket folds all blocks' candidates; nobody waits for anybody
        if (threadIdx.x == 0) s_last = atomicAdd(p.am.count, 1u) == gridDim.x - 1u;
        __syncthreads();
        if (s_last) {
            __threadfence();
            if (warp < (uint32_t)M) {                  // one warp per batch row
                float best = kArgmaxLowest;
                uint32_t at = 0xFFFFFFFFu;
                for (uint32_t b = lane; b < gridDim.x; b += 32u)
                    argmax_take(__ldcg(p.am.block_val + (size_t)b * M + warp), __ldcg(p.am.block_idx + (size_t)b * M + warp), best, at);
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
                    const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, at, off);
                    argmax_take(ov, oi, best, at);
                }
                if (lane == 0u) {
                    p.am.out_idx[warp] = at == 0xFFFFFFFFu ? p.am.index_base : at;   // a row of NaNs: its first column
                    if (p.am.out_val) p.am.out_val[warp] = best;
                }
            }
            if (threadIdx.x == 0) *p.am.count = 0u;    // ready for the next launch
        }
    }
}

// Any K, any alignment, any dtype mix: one warp per output column, scalar loads.
// Used when K is not a multiple of the vector width or a pointer is not 16-byte
// aligned (vAi's slab kernel has the same split: linear-slab.comp:98-116).
__global__ void __launch_bounds__(kThreads) gemv_generic_kernel(const GemvParams p)
{
    const LinearArgs& a = p.a;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t col = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t H = p.H;
    if (col >= H) return;
    const bool gate = a.gate_fuse != 0;
    const EpilogueArgs ep = make_epilogue_args(a);
    float acc[8], acc2[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) { acc[m] = 0.0f; acc2[m] = 0.0f; }
    for (uint32_t k = lane; k < a.K; k += 32u) {
        const float w = load_as_f32(a.W, a.w_dtype, (size_t)col * a.K + k);
        const float w2 = gate ? load_as_f32(a.W, a.w_dtype, (size_t)(H + col) * a.K + k) : 0.0f;
#pragma unroll
        for (int m = 0; m < 8; ++m)
            if ((uint32_t)m < a.M) {
                const float x = load_as_f32(a.I, a.i_dtype, (size_t)m * a.K + k);
                acc[m] = fmaf(w, x, acc[m]);
                acc2[m] = fmaf(w2, x, acc2[m]);
            }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            acc[m] += __shfl_xor_sync(0xFFFFFFFFu, acc[m], off);
            acc2[m] += __shfl_xor_sync(0xFFFFFFFFu, acc2[m], off);
        }
#pragma unroll
    for (int m = 0; m < 8; ++m)
        if (lane == (uint32_t)m && (uint32_t)m < a.M) {
            const size_t flat = (size_t)m * H + col;
            const float v = gate ? finish_gated(ep, acc[m], acc2[m], col, H, flat) : finish_output(ep, acc[m], flat);
            store_from_f32(a.O, a.o_dtype, flat, v);
        }
}

template <typename TW, int M, int R, int U = 2>
cudaError_t launch_one(const GemvParams& p, const GemvConfig& cfg, cudaStream_t stream)
{
    auto kern = gemv_kernel<TW, M, R, U>;
    static SmemOptIn optin;
    if (cudaError_t e = optin.ensure(kern, 100 * 1024); e != cudaSuccess) return e;
    // Programmatic stream serialization: this launch may begin while the kernel ahead
    // of it in the stream drains; gemv_kernel itself waits (dependency_wait) before it
    // reads anything that kernel produced.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)cfg.grid);
    lc.blockDim = dim3(kThreads);
    lc.dynamicSmemBytes = cfg.smem;
    lc.stream = stream;
    lc.attrs = attr;
    lc.numAttrs = cfg.plain_launch ? 0 : 1;
#ifdef VAICU_GEMV_TRACE
    GemvParams traced = p;
    traced.trace_id = g_gemv_trace_next++;
    return cudaLaunchKernelEx(&lc, kern, traced);
#else
    return cudaLaunchKernelEx(&lc, kern, p);
#endif
}

#ifdef VAICU_GEMV_TRACE
extern "C" __attribute__((visibility("default"))) int vaicu_debug_gemv_trace(unsigned long long* out, unsigned* next, int reset)
{
    if (next) *next = g_gemv_trace_next;
    if (reset) { g_gemv_trace_next = 0; return 0; }
    return (int)cudaMemcpyFromSymbol(out, g_gemv_trace, sizeof(g_gemv_trace));
}
#endif

template <typename TW>
cudaError_t launch_typed(const GemvParams& p, const GemvConfig& cfg, cudaStream_t stream)
{
    const bool r4 = cfg.rows_per_warp == 4;
    switch (p.a.M) {
    case 1:
        if (cfg.unroll == 4) return r4 ? launch_one<TW, 1, 4, 4>(p, cfg, stream) : launch_one<TW, 1, 2, 4>(p, cfg, stream);
        return r4 ? launch_one<TW, 1, 4, 2>(p, cfg, stream) : launch_one<TW, 1, 2, 2>(p, cfg, stream);
    case 2: return r4 ? launch_one<TW, 2, 4>(p, cfg, stream) : launch_one<TW, 2, 2>(p, cfg, stream);
    case 3: return r4 ? launch_one<TW, 3, 4>(p, cfg, stream) : launch_one<TW, 3, 2>(p, cfg, stream);
    case 4: return r4 ? launch_one<TW, 4, 4>(p, cfg, stream) : launch_one<TW, 4, 2>(p, cfg, stream);
    case 5: return launch_one<TW, 5, 2>(p, cfg, stream);
    case 6: return launch_one<TW, 6, 2>(p, cfg, stream);
    case 7: return launch_one<TW, 7, 2>(p, cfg, stream);
    case 8: return launch_one<TW, 8, 2>(p, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace

// Shape -> launch geometry (the analogue of ggmlSlabWgSize, vAi linear.h:655-663:
// deep-K layers with few rows get their K split over several warps).
GemvConfig choose_gemv(const LinearArgs& a, int sm_count, bool ptrs_aligned16, const vaicu_linear_tuning* tuning)
{
    GemvConfig c{};
    c.plain_launch = (tuning && tuning->gemv_plain_launch) ? 1 : 0;
    const int vec = a.w_dtype == VAICU_DTYPE_F32 ? 4 : 8;
    const uint32_t H = a.gate_fuse ? a.N / 2u : a.N;
    c.vectorized = ptrs_aligned16 && (a.K % (uint32_t)vec == 0u) && a.M >= 1u && a.M <= 8u;
    if (!c.vectorized) {
        c.rows_per_warp = 1; c.k_warps = 1; c.smem = 0;
        c.grid = (int)((H + kWarps - 1u) / kWarps);
        return c;
    }
    // Blocks resident at once: 2 per SM (launch bounds).  One
    // block-task = (8 / ks) row groups of R rows, K split over ks warps.  Wanted: all
    // tasks in flight together (no ragged second round), and at least half the
    // resident slots used; so few rows get a smaller R and a deeper K split, while
    // every warp keeps two 16-byte steps.
    // M = 1 comes in two depths: U = 2 k-steps in flight at 3 blocks per SM (96 KB per SM), or U = 4 at
    // 2 blocks per SM (128 KB per SM).  A layer whose weights the resident blocks request in one trip at
    // U = 2 (14.5 MB on 148 SMs) gains nothing from the deeper form and loses resident slots to it; a larger
    // layer is bound by the bytes in flight (measured in the recorded Llama-3.2-1B step: gate|value and down
    // at U = 4 take 9 us off 529, the lm_head is unchanged, o at U = 4 adds 11 us).
    const uint64_t one_trip = (uint64_t)sm_count * 3u * (uint64_t)kThreads * 2u * 4u * 16u;
    const uint64_t weight_bytes = (uint64_t)a.N * a.K * (a.w_dtype == VAICU_DTYPE_F32 ? 4u : 2u);
    c.unroll = (a.M == 1u && weight_bytes > one_trip) ? 4 : 2;
    if (a.M == 1u && tuning && (tuning->gemv_unroll == 2 || tuning->gemv_unroll == 4)) c.unroll = tuning->gemv_unroll;
    const uint32_t capacity = (uint32_t)sm_count * ((a.M == 1u && c.unroll == 2) ? 3u : 2u);
    // Measured: a deeper K split than needed is costly (lm_head 76 -> 108 us with ks = 2:
    // every pass then ends in a block-wide fold), so K is split only until about half
    // the resident slots are used, and R shrinks only when even that cannot be reached.
    int R = a.M <= 4u ? 4 : 2, ks = 1;
    uint32_t best_tasks = 0;
    for (int r = (a.M <= 4u ? 4 : 2); r >= 2; r -= 2) {
        const uint32_t cols_r = a.gate_fuse ? (uint32_t)r / 2u : (uint32_t)r;
        const uint32_t groups_r = (H + cols_r - 1u) / cols_r;
        bool done = false;
        for (int k = 1; k <= kWarps; k *= 2) {
            if (k > 1 && a.K / (uint32_t)(k * 32 * vec) < 2u) break;
            const uint32_t tasks = (groups_r + (uint32_t)(kWarps / k) - 1u) / (uint32_t)(kWarps / k);
            if (tasks > best_tasks) { best_tasks = tasks; R = r; ks = k; }
            if (tasks * 2u >= capacity) { done = true; break; }
        }
        if (done) break;
    }
    {
        // Between one and two rounds the equal-pass grid leaves ~40 % of the resident slots
        // empty (gate|value of Llama-1B: 512 tasks -> 256 blocks of 2 passes).  One more K
        // doubling then fills more slots (1024 tasks -> 342 blocks of 3 passes: 14.7 -> 13.1 us
        // measured); doubling further loses again to the per-pass fold.
        const uint32_t cols_r = a.gate_fuse ? (uint32_t)R / 2u : (uint32_t)R;
        const uint32_t groups_r = (H + cols_r - 1u) / cols_r;
        auto resident = [&](int k) {
            const uint32_t tasks = (groups_r + (uint32_t)(kWarps / k) - 1u) / (uint32_t)(kWarps / k);
            const uint32_t rounds_k = (tasks + capacity - 1u) / capacity;
            return (tasks + rounds_k - 1u) / rounds_k;
        };
        if (ks < kWarps && a.K / (uint32_t)(2 * ks * 32 * vec) >= 2u && resident(ks) * 10u < capacity * 7u &&
            resident(2 * ks) > resident(ks))
            ks *= 2;
    }
    if (tuning) {   // a caller's overrides
        if (tuning->gemv_rows == 2 || (tuning->gemv_rows == 4 && a.M <= 4u)) R = tuning->gemv_rows;
        const int v = tuning->gemv_k_warps;
        if (v == 1 || v == 2 || v == 4 || v == 8) ks = v;
    }
    const uint32_t cols = a.gate_fuse ? (uint32_t)R / 2u : (uint32_t)R;
    const uint32_t groups = (H + cols - 1u) / cols;
    c.rows_per_warp = R;
    c.k_warps = ks;
    const uint32_t budget_floats = (96u * 1024u) / 4u / a.M;
    uint32_t k_chunk = (budget_floats / 256u) * 256u;
    const uint32_t k_round = ((a.K + 255u) / 256u) * 256u;
    if (k_chunk > k_round) k_chunk = k_round;
    if (a.M == 1u) k_chunk = 0;   // M = 1 reads its activations from global memory: only the fold buffer
    c.smem = ((size_t)a.M * k_chunk + (size_t)kWarps * R * a.M) * sizeof(float);
    const uint32_t rg = (uint32_t)kWarps / (uint32_t)ks;
    const uint32_t nblocks = (groups + rg - 1u) / rg;
    // equal passes per block: with more tasks than resident slots, shrink the grid so
    // that every block runs the same number of passes instead of leaving a short tail
    const uint32_t rounds = (nblocks + capacity - 1u) / capacity;
    c.grid = (int)((nblocks + rounds - 1u) / rounds);
    if (tuning && tuning->gemv_grid > 0) c.grid = tuning->gemv_grid < (int)nblocks ? tuning->gemv_grid : (int)nblocks;
    return c;
}

cudaError_t launch_gemv_group(const LinearArgs& a, const GemvConfig& cfg, uint32_t nseg, const uint32_t* rows,
                              const void* const* w, void* const* o, cudaStream_t stream)
{
    if (nseg < 2u || nseg > 3u || !cfg.vectorized || a.gate_fuse) return cudaErrorInvalidValue;
    GemvParams p{};
    p.a = a;
    p.H = a.N;
    p.nseg = nseg;
    uint32_t total = 0;
    for (uint32_t i = 0; i < 4u; ++i) p.seg_begin[i] = 0xFFFFFFFFu;
    for (uint32_t i = 0; i < nseg; ++i) {
        p.seg_begin[i] = total;
        p.seg_w[i] = w[i];
        p.seg_o[i] = o[i];
        total += rows[i];
    }
    p.seg_begin[nseg] = total;
    if (total != a.N) return cudaErrorInvalidValue;
    p.cols_per_warp = (uint32_t)cfg.rows_per_warp;
    p.k_warps = (uint32_t)cfg.k_warps;
    const uint32_t budget_floats = (96u * 1024u) / 4u / a.M;
    uint32_t k_chunk = (budget_floats / 256u) * 256u;
    const uint32_t k_round = ((a.K + 255u) / 256u) * 256u;
    if (k_chunk > k_round) k_chunk = k_round;
    p.k_chunk = a.M == 1u ? k_round : k_chunk;
    p.k_pad = a.M == 1u ? 0u : k_chunk;
    switch (a.w_dtype) {
    case VAICU_DTYPE_F32: return launch_typed<float>(p, cfg, stream);
    case VAICU_DTYPE_F16: return launch_typed<__half>(p, cfg, stream);
    case VAICU_DTYPE_BF16: return launch_typed<__nv_bfloat16>(p, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemv(const LinearArgs& a, const GemvConfig& cfg, cudaStream_t stream, const GemvArgmax* argmax)
{
    GemvParams p{};
    p.a = a;
    p.H = a.gate_fuse ? a.N / 2u : a.N;
    if (argmax) {
        if (!cfg.vectorized || a.gate_fuse) return cudaErrorInvalidValue;
        p.am = *argmax;
    }
    if (!cfg.vectorized) {
        gemv_generic_kernel<<<cfg.grid, kThreads, 0, stream>>>(p);
        return cudaGetLastError();
    }
    p.cols_per_warp = a.gate_fuse ? (uint32_t)cfg.rows_per_warp / 2u : (uint32_t)cfg.rows_per_warp;
    p.k_warps = (uint32_t)cfg.k_warps;
    const uint32_t budget_floats = (96u * 1024u) / 4u / a.M;
    uint32_t k_chunk = (budget_floats / 256u) * 256u;
    const uint32_t k_round = ((a.K + 255u) / 256u) * 256u;
    if (k_chunk > k_round) k_chunk = k_round;
    p.k_chunk = a.M == 1u ? k_round : k_chunk;   // M = 1: one span, nothing staged
    p.k_pad = a.M == 1u ? 0u : k_chunk;
    switch (a.w_dtype) {
    case VAICU_DTYPE_F32: return launch_typed<float>(p, cfg, stream);
    case VAICU_DTYPE_F16: return launch_typed<__half>(p, cfg, stream);
    case VAICU_DTYPE_BF16: return launch_typed<__nv_bfloat16>(p, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace vaicu
