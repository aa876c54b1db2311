// Tensor-core kernel of the Linear path for M > 8: D = A . B^T with both
// operands K-major 16-bit (bf16 or fp16), fp32 accumulation in tensor memory.
//
// Stands where vAi's cooperative-matrix tile kernel does
// (vai/shaders/linear-cm-nv.comp, selected in vai/nodes/linear.h:2436), with the
// bias / epilogue / residual / scale that the reference leaves to a second pass
// (vai/shaders/linear-reduce.comp) fused into the store, and optionally the
// GatedMul that follows a gate|value Linear (vai/nodes/gated-mul.h:9-20).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0    one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//             into a ring of shared-memory stages, signalled through mbarriers;
//   warp 1    allocates tensor memory; one lane issues tcgen05.mma
//             (cta_group::1, M = 128, N = bn, K = 16) and commits each stage back
//             to the producer and each finished tile to the epilogue;
//   warps 2-5 read the accumulator with tcgen05.ld (each warp owns 32 TMEM
//             lanes), apply the epilogue and store.  Two accumulator buffers let
//             the epilogue of tile i overlap the main loop of tile i+1.
// "rows" operand A sits on the UMMA M axis (128 TMEM lanes), "cols" operand B on
// the UMMA N axis (TMEM columns).  Large M: A = activations, B = weights.
// Small M ("swap"): A = weights, B = activations, so a 128-row slab of W is
// streamed once and the batch rides on N.
// For M > 128 a second kernel (tc_gemm_pair_kernel, below) runs the same pipeline on
// clusters of two CTAs with tcgen05.mma.cta_group::2.
// Every wait is bounded; on expiry the kernel records a status word and leaves.
#include <cuda.h>

#include "common.cuh"
#include "tc_gemm.h"

namespace vaicu {

namespace {

constexpr uint32_t BLOCK_K = 64;          // 64 x 2 bytes = one 128-byte swizzle row
constexpr uint32_t UMMA_K = 16;
constexpr uint32_t TILE_ROWS = 128;       // UMMA M
constexpr uint32_t kTcThreads = 192;        // producer warp, MMA warp, 4 epilogue warps
constexpr uint32_t kTcThreadsSwap = 320;    // swapped kernel: 8 epilogue warps, two per quarter of the TMEM lanes
constexpr uint32_t kSpinLimit = 1u << 24; // bounded waits (each probe may sleep in hardware)

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another role already
// gave up (abort flag), so that no role spins forever.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag)
{
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1u;
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes,
// stored with the 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO),
// LBO is unused for swizzled K-major layouts (encoded 1), descriptor version 1,
// layout type 2 (SWIZZLE_128B).  The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr)
{
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

// ---- epilogue store helpers -----------------------------------------------
__device__ __forceinline__ void store16(void* O, int o_dtype, size_t flat, const float* v, bool vec_ok)
{
    if (vec_ok) {
        if (o_dtype == VAICU_DTYPE_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(O) + flat);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
            uint32_t w[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (o_dtype == VAICU_DTYPE_F16) {
                    __half2 h = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
                    w[q] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
                    w[q] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(O) + flat);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
    }
}

// Epilogue functions with the reference's formulas (vAi
// vai/shaders/common/activation.h:19-58) on the fast exp / divide units; the tanh
// is written through exp.  Sixteen values at a time with the switch outside the
// loops: each case is straight-line code, so the epilogue warps fetch one short
// path instead of a branch tree per element.
__device__ __forceinline__ void act16(int code, float* v)
{
    switch (code) {
    case VAICU_EPILOGUE_RELU:
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] = fmaxf(v[c], 0.0f);
        break;
    case VAICU_EPILOGUE_GELU:
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const float x = v[c], y = x * 0.707106781186547524400844f;
            const float t = __fdividef(1.0f, 1.0f + 0.3275911f * fabsf(y));
            const float pl = ((((1.061405429f * t - 1.453152027f) * t + 1.421413741f) * t - 0.284496736f) * t + 0.254829592f) * t;
            v[c] = 0.5f * x * (1.0f + copysignf(1.0f - pl * __expf(-y * y), y));
        }
        break;
    case VAICU_EPILOGUE_GELU_TANH:
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const float x = v[c];
            const float u = 0.797884560802865355879892f * (x + 0.044715f * x * x * x);
            v[c] = 0.5f * x * (2.0f - __fdividef(2.0f, __expf(2.0f * u) + 1.0f));
        }
        break;
    case VAICU_EPILOGUE_SILU:
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] = __fdividef(v[c], 1.0f + __expf(-v[c]));
        break;
    case VAICU_EPILOGUE_SIGMOID:
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] = __fdividef(1.0f, 1.0f + __expf(-v[c]));
        break;
    default: break;
    }
}

// f[c] = element idx0 + c of a dtype'd array, c < 16; elements at or past n_valid
// repeat the last valid one (their results are never stored).
__device__ __forceinline__ void load16(const void* base, int dt, size_t idx0, uint32_t n_valid, float* f)
{
    const uint32_t esz = dtype_size(dt);
    const bool vec = n_valid >= 16u && (((reinterpret_cast<uintptr_t>(base) + idx0 * esz) & 15u) == 0);
    if (dt == VAICU_DTYPE_F32) {
        const float* s = reinterpret_cast<const float*>(base) + idx0;
        if (vec) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 t = reinterpret_cast<const float4*>(s)[q];
                f[4 * q] = t.x; f[4 * q + 1] = t.y; f[4 * q + 2] = t.z; f[4 * q + 3] = t.w;
            }
        } else {
#pragma unroll
            for (uint32_t c = 0; c < 16u; ++c) f[c] = s[c < n_valid ? c : n_valid - 1u];
        }
    } else {
        const uint16_t* s = reinterpret_cast<const uint16_t*>(base) + idx0;
        uint32_t w[8];
        if (vec) {
            const uint4 t0 = reinterpret_cast<const uint4*>(s)[0], t1 = reinterpret_cast<const uint4*>(s)[1];
            w[0] = t0.x; w[1] = t0.y; w[2] = t0.z; w[3] = t0.w; w[4] = t1.x; w[5] = t1.y; w[6] = t1.z; w[7] = t1.w;
        } else {
#pragma unroll
            for (uint32_t q = 0; q < 8u; ++q) {
                const uint32_t i0 = 2u * q < n_valid ? 2u * q : n_valid - 1u;
                const uint32_t i1 = 2u * q + 1u < n_valid ? 2u * q + 1u : n_valid - 1u;
                w[q] = (uint32_t)s[i0] | ((uint32_t)s[i1] << 16);
            }
        }
        if (dt == VAICU_DTYPE_F16) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                f[2 * q] = t.x; f[2 * q + 1] = t.y;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                f[2 * q] = __uint_as_float(w[q] << 16);
                f[2 * q + 1] = __uint_as_float(w[q] & 0xFFFF0000u);
            }
        }
    }
}

// Sixteen residual values of one output row, requested early and unpacked when the accumulators are
// ready: the epilogue of the CTA-pair kernel asks for the next chunk's residual before it works on the
// current one, so that the load's latency is not paid once per chunk.
struct ResRaw {
    uint4 q[4];
    bool valid;
};
__device__ __forceinline__ void res_issue(const TcParams& p, uint32_t m, uint32_t j0, uint32_t out_cols, ResRaw& r)
{
    r.valid = false;
    if (p.res_mode != OPERAND_FULL || p.partial || m >= p.M || j0 + 16u > out_cols) return;
    const uint32_t osz = dtype_size(p.o_dtype);
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.res) + ((size_t)m * out_cols + j0) * osz;
    if (addr & 15u) return;
    const uint4* s = reinterpret_cast<const uint4*>(addr);
    r.q[0] = s[0];
    r.q[1] = s[1];
    if (osz == 4u) { r.q[2] = s[2]; r.q[3] = s[3]; }
    r.valid = true;
}
__device__ __forceinline__ void res_unpack(int dt, const ResRaw& r, float* t)
{
    if (dt == VAICU_DTYPE_F32) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            t[4 * k] = __uint_as_float(r.q[k].x); t[4 * k + 1] = __uint_as_float(r.q[k].y);
            t[4 * k + 2] = __uint_as_float(r.q[k].z); t[4 * k + 3] = __uint_as_float(r.q[k].w);
        }
        return;
    }
    const uint32_t w[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (dt == VAICU_DTYPE_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            t[2 * k] = f.x; t[2 * k + 1] = f.y;
        } else {
            t[2 * k] = __uint_as_float(w[k] << 16); t[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
    }
}

// 16 consecutive output columns [j0, j0+16) of activation row m (kernel without swap).
// v: accumulators (gate half with GATE), u: value-half accumulators.
template <bool GATE>
__device__ __forceinline__ void finish_row16(const TcParams& p, float* v, float* u, uint32_t m, uint32_t j0,
                                             uint32_t out_cols, uint32_t n_valid, const ResRaw* pre = nullptr)
{
    const size_t flat0 = (size_t)m * out_cols + j0;
    float t[16];
    if (p.bias_mode == OPERAND_PER_COLUMN) {
        load16(p.bias, p.b_dtype, j0, n_valid, t);
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] += t[c];
        if (GATE) {
            load16(p.bias, p.b_dtype, (size_t)p.H + j0, n_valid, t);
#pragma unroll
            for (int c = 0; c < 16; ++c) u[c] += t[c];
        }
    } else if (p.bias_mode != OPERAND_NONE) {   // [M,N] or repeating tables (never with GATE)
        for (uint32_t c = 0; c < 16u; ++c) {
            const size_t i = (size_t)m * p.N + j0 + (c < n_valid ? c : n_valid - 1u);
            v[c] += load_as_f32(p.bias, p.b_dtype, p.bias_mode == OPERAND_MODULO ? i % p.bias_elems : i);
        }
    }
    if (p.res_mode == OPERAND_FULL && pre && pre->valid) res_unpack(p.o_dtype, *pre, t);
    else if (p.res_mode == OPERAND_FULL) load16(p.res, p.o_dtype, flat0, n_valid, t);
    else if (p.res_mode == OPERAND_PER_COLUMN) load16(p.res, p.o_dtype, j0, n_valid, t);
    else if (p.res_mode == OPERAND_MODULO)
        for (uint32_t c = 0; c < 16u; ++c) t[c] = load_as_f32(p.res, p.o_dtype, (flat0 + (c < n_valid ? c : n_valid - 1u)) % p.res_elems);
    const bool before = p.res_mode != OPERAND_NONE && p.residual_order == VAICU_RESIDUAL_BEFORE_EPILOGUE;
    const bool after = p.res_mode != OPERAND_NONE && !before;
    if (before) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] += t[c];
    }
    act16(p.epilogue, v);
    if (GATE) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] *= u[c];
    }
    if (p.scale != 1.0f) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] *= p.scale;
    }
    if (after) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] += t[c];
    }
}

// Swapped kernel: this thread owns weight row n; the 16 values are activation rows
// m0 .. m0+15 of that output column.
template <bool GATE>
__device__ __forceinline__ void finish_col16(const TcParams& p, float* v, float* u, uint32_t n, uint32_t m0,
                                             uint32_t out_cols, float bias_n, float bias_up)
{
    float t[16];
    if (p.bias_mode == OPERAND_PER_COLUMN) {
#pragma unroll
        for (int c = 0; c < 16; ++c) { v[c] += bias_n; if (GATE) u[c] += bias_up; }
    } else if (p.bias_mode != OPERAND_NONE) {
        for (uint32_t c = 0; c < 16u; ++c) {
            const uint32_t m = m0 + c < p.M ? m0 + c : p.M - 1u;
            const size_t i = (size_t)m * p.N + n;
            v[c] += load_as_f32(p.bias, p.b_dtype, p.bias_mode == OPERAND_MODULO ? i % p.bias_elems : i);
        }
    }
    if (p.res_mode == OPERAND_FULL) {
        // the common case: one residual per output, 16 independent loads down this thread's column
#pragma unroll
        for (uint32_t c = 0; c < 16u; ++c) {
            const uint32_t m = m0 + c < p.M ? m0 + c : p.M - 1u;
            t[c] = load_as_f32(p.res, p.o_dtype, (size_t)m * out_cols + n);
        }
    } else if (p.res_mode == OPERAND_PER_COLUMN) {
        const float r = load_as_f32(p.res, p.o_dtype, n);
#pragma unroll
        for (uint32_t c = 0; c < 16u; ++c) t[c] = r;
    } else if (p.res_mode != OPERAND_NONE) {
        for (uint32_t c = 0; c < 16u; ++c) {
            const uint32_t m = m0 + c < p.M ? m0 + c : p.M - 1u;
            t[c] = load_as_f32(p.res, p.o_dtype, ((size_t)m * out_cols + n) % p.res_elems);
        }
    }
    const bool before = p.res_mode != OPERAND_NONE && p.residual_order == VAICU_RESIDUAL_BEFORE_EPILOGUE;
    const bool after = p.res_mode != OPERAND_NONE && !before;
    if (before) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] += t[c];
    }
    act16(p.epilogue, v);
    if (GATE) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] *= u[c];
    }
    if (p.scale != 1.0f) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] *= p.scale;
    }
    if (after) {
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] += t[c];
    }
}

// Unswapped kernel: 16 finished dot products (v; u = the value half with GATE) of activation row m,
// output columns [j0, j0 + 16): bias / epilogue / residual / scale, then the stores.
template <bool GATE>
__device__ __forceinline__ void emit_rows16(const TcParams& p, float* v, float* u, uint32_t m, uint32_t j0, uint32_t out_cols,
                                            uint32_t osz, const ResRaw* pre = nullptr)
{
    const uint32_t n_valid = out_cols - j0 < 16u ? out_cols - j0 : 16u;
    finish_row16<GATE>(p, v, u, m, j0, out_cols, n_valid, pre);
    // O may be a column slab of wider destinations (ldo, col0), one per GPU; a row-parallel run
    // sends the row to the one GPU that owns it
    if (p.grp_t1 != kNoGroup) {
        // a group of plain Linears over the same activations (CTA-pair kernel): columns [0, N) are the members'
        // outputs side by side, whole tiles each; this chunk goes to the member that owns column j0
        const uint32_t n1 = p.grp_t1 * p.bn, n2 = p.grp_t2 == kNoGroup ? p.N : p.grp_t2 * p.bn;
        const uint32_t j = j0 >= n2 ? 2u : (j0 >= n1 ? 1u : 0u);
        const uint32_t first = j == 2u ? n2 : (j == 1u ? n1 : 0u);
        const uint32_t width = (j == 0u ? n1 : (j == 1u ? n2 : p.N)) - first;
        const size_t at = (size_t)m * width + (j0 - first);
        if (n_valid == 16u && ((at * osz) % 16u == 0u)) store16(p.dst[j], p.o_dtype, at, v, true);
        else
            for (uint32_t c = 0; c < n_valid; ++c) store_from_f32(p.dst[j], p.o_dtype, at + c, v[c]);
        return;
    }
    uint32_t owner;
    size_t row;
    output_row(p, m, owner, row);
    const size_t flat0 = row * p.ldo + p.col0 + j0;
    const bool vec_ok = n_valid == 16u && (((size_t)flat0 * osz) % 16u == 0u) && p.o_aligned16;
    for (uint32_t d = 0; d < p.n_dst; ++d) {
        if (owner != 0xFFFFFFFFu && d != owner) continue;
        void* dst = p.n_dst == 1u ? p.O : p.dst[d];
        if (vec_ok) store16(dst, p.o_dtype, flat0, v, true);
        else
            for (uint32_t c = 0; c < n_valid; ++c) store_from_f32(dst, p.o_dtype, flat0 + c, v[c]);
    }
}

// Swapped kernel: this thread owns output column n; v holds its dot products with activation rows
// m0 .. m0 + 15: bias / epilogue / residual / scale, then the (column-strided) stores.
template <bool GATE>
__device__ __forceinline__ void emit_cols16(const TcParams& p, float* v, float* u, uint32_t n, uint32_t m0, uint32_t out_cols,
                                            float bias_n, float bias_up)
{
    finish_col16<GATE>(p, v, u, n, m0, out_cols, bias_n, bias_up);
    if (p.rs_rows) {                       // row-parallel run: each activation row goes to its owner's staging
        for (uint32_t c = 0; c < 16u; ++c) {
            if (m0 + c >= p.M) break;
            uint32_t owner;
            size_t row;
            output_row(p, m0 + c, owner, row);
            store_from_f32(p.dst[owner], p.o_dtype, row * p.ldo + p.col0 + n, v[c]);
        }
        return;
    }
    for (uint32_t d = 0; d < p.n_dst; ++d) {
        void* dst = p.n_dst == 1u ? p.O : p.dst[d];
        if (p.o_dtype == VAICU_DTYPE_F32) {
            float* O = reinterpret_cast<float*>(dst);
#pragma unroll
            for (uint32_t c = 0; c < 16u; ++c)
                if (m0 + c < p.M) O[(size_t)(m0 + c) * p.ldo + p.col0 + n] = v[c];
        } else if (p.o_dtype == VAICU_DTYPE_F16) {
            __half* O = reinterpret_cast<__half*>(dst);
#pragma unroll
            for (uint32_t c = 0; c < 16u; ++c)
                if (m0 + c < p.M) O[(size_t)(m0 + c) * p.ldo + p.col0 + n] = __float2half_rn(v[c]);
        } else {
            __nv_bfloat16* O = reinterpret_cast<__nv_bfloat16*>(dst);
#pragma unroll
            for (uint32_t c = 0; c < 16u; ++c)
                if (m0 + c < p.M) O[(size_t)(m0 + c) * p.ldo + p.col0 + n] = __float2bfloat16_rn(v[c]);
        }
    }
}

// Unswapped epilogue for 16 accumulator columns starting at c0 of one 128-row block:
// this thread owns activation row m.  r0 / r1 hold the raw accumulators (r1: the value
// half with GATE).  Either raw split-K partials or the finished outputs are stored.
template <bool GATE>
__device__ __forceinline__ void store_rows16(const TcParams& p, const uint32_t* r0, const uint32_t* r1, uint32_t m,
                                             uint32_t tb, uint32_t c0, uint32_t z, uint32_t out_cols, uint32_t osz,
                                             const ResRaw* pre = nullptr)
{
    const uint32_t bn = p.bn;
    if (p.partial) {
        // split-K: raw fp32 partial sums, [z][M][N]; epilogue runs in the reduce pass
        float* P = p.partial + (size_t)z * p.M * p.N;
        if (m < p.M) {
#pragma unroll
            for (uint32_t c = 0; c < 16u; ++c) {
                const uint32_t col = c0 + c;
                if (GATE) {
                    const uint32_t j = tb * (bn / 2u) + col;
                    if (j < p.H) {
                        P[(size_t)m * p.N + j] = __uint_as_float(r0[c]);
                        P[(size_t)m * p.N + p.H + j] = __uint_as_float(r1[c]);
                    }
                } else {
                    const uint32_t n = tb * bn + col;
                    if (n < p.N) P[(size_t)m * p.N + n] = __uint_as_float(r0[c]);
                }
            }
        }
        return;
    }
    const uint32_t j0 = (GATE ? tb * (bn / 2u) : tb * bn) + c0;
    if (m < p.M && j0 < out_cols) {
        float v[16], u[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) { v[c] = __uint_as_float(r0[c]); u[c] = GATE ? __uint_as_float(r1[c]) : 0.0f; }
        emit_rows16<GATE>(p, v, u, m, j0, out_cols, osz, pre);
    }
}

}  // namespace

// Forms that address another CTA of the cluster.
namespace {
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of this CTA's shared-memory location `local` inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr)
{
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}
}  // namespace

#ifdef VAICU_TC_TRACE
// Development aid (not built by default): phase time stamps of every CTA of the single-CTA kernel.
__device__ unsigned long long g_tc_trace[256 * 16];
__device__ __forceinline__ void tc_trace(uint32_t slot)
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (blockIdx.x < 256u) g_tc_trace[blockIdx.x * 16u + slot] = t;
}
#define TC_TRACE(slot) tc_trace(slot)
#else
#define TC_TRACE(slot)
#endif

// SWAP: A (TMEM lanes) = weights, B (TMEM columns) = activations.
// GATE: fused Linear + GatedMul.  Non-swap: the B stage holds bn/2 gate rows then
//       bn/2 value rows; swap: the A stage holds 128 gate rows then 128 value rows
//       and two MMAs per k-step fill two accumulators.
template <bool SWAP, bool GATE>
__global__ void __launch_bounds__(SWAP ? kTcThreadsSwap : kTcThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_a1, const __grid_constant__ CUtensorMap tmap_a2, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle atoms
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t bn = p.bn;
    if (threadIdx.x == 0) TC_TRACE(0);
    // wide: two 128-row A boxes per stage and two MMAs per k-step give a 256-row tile;
    // the weights' B tile is then fetched once per 256 rows instead of once per 128,
    // which is what the operand traffic from L2 allows at full tensor rate.
    const bool wide = !SWAP && p.wide != 0u;
    const uint32_t a_boxes = ((GATE && SWAP) || wide) ? 2u : 1u;
    // Swapped: a weight tile may hold fewer than 128 rows (p.tile_rows, a multiple of 8), so that a layer
    // with fewer than one 128-row tile per SM still spreads over all SMs.  The MMA stays 128 rows tall; the
    // rows of the slot that the copy does not fill are whatever the slot held, and the accumulator lanes
    // they feed are never read.
    const uint32_t tile_rows = SWAP ? p.tile_rows : TILE_ROWS;
    const uint32_t a_rows = wide ? 2u * TILE_ROWS : tile_rows;   // rows per tile on the A side
    const uint32_t a_bytes = a_boxes * TILE_ROWS * BLOCK_K * 2u;
    const uint32_t b_bytes = bn * BLOCK_K * 2u;
    const uint32_t stage_bytes = a_bytes + b_bytes;        // multiple of 1024 (bn % 8 == 0)
    const uint32_t tx_bytes = a_boxes * tile_rows * BLOCK_K * 2u + b_bytes;     // what the copies of one stage deliver
    const uint32_t stages = p.stages;
    const uint32_t acc_cols = a_boxes * bn;            // TMEM columns per accumulator buffer
    const uint32_t acc_bufs = p.acc_bufs;              // 2: epilogue overlaps the next tile; 1: 512 columns in use

    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
    uint64_t* empty_bar = full_bar + stages;
    uint64_t* acc_full = empty_bar + stages;      // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint64_t* fold_in = acc_empty + 2;            // split-K fold: the four epilogue warps have written their partials
    uint64_t* fold_out = fold_in + 1;             // ... and the ticket for this tile has been drawn
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fold_out + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* fold_flag = tmem_slot + 2;     // epilogue warps: "this CTA folds the tile's splits"
    // Split-K folded inside a cluster (p.cfold CTAs = the K splits of one tile): every CTA leaves its raw
    // accumulator here, [bn columns][128 lanes] fp32, for its cluster mates to read.
    float* red = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes + 256u);
    const bool cfold = SWAP && !GATE && p.cfold != 0u;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        // epilogue warps: 4, or 8 that share each quarter of the accumulator's lanes by column chunks (swapped
        // kernel: its CTAs often hold a single tile, whose epilogue nothing overlaps)
        const uint32_t epi_warps = (blockDim.x >> 5) - 2u;
        for (uint32_t b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], epi_warps); }
        mbar_init(fold_in, epi_warps);
        mbar_init(fold_out, 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (SWAP && !GATE && p.grp_t1 != kNoGroup) {
            prefetch_tmap(&tmap_a1);
            prefetch_tmap(&tmap_a2);
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) TC_TRACE(1);

    const uint32_t num_work = p.num_tiles * p.splits;

    // The launch after this one may begin its prologue now (it waits before it touches our results).
    launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // One k-block of one operand into its stage.  "A" sits on the UMMA M axis, "B" on N.
            auto load_a = [&](uint32_t st, uint32_t kb, uint32_t ta) {
                uint8_t* sa = smem + (size_t)st * stage_bytes;
                const int32_t kx = (int32_t)(kb * BLOCK_K);
                if (SWAP && !GATE && ta >= p.grp_t1) {
                    // a group of Linears over the same activations: the weight tiles of the second and
                    // third member come from their own tensors (members are whole numbers of tiles)
                    const bool third = ta >= p.grp_t2;
                    tma_load_2d(sa, third ? &tmap_a2 : &tmap_a1, &full_bar[st], kx,
                                (int32_t)((ta - (third ? p.grp_t2 : p.grp_t1)) * a_rows));
                    return;
                }
                tma_load_2d(sa, &tmap_a, &full_bar[st], kx, (int32_t)(ta * a_rows));
                if (a_boxes == 2u)
                    tma_load_2d(sa + TILE_ROWS * BLOCK_K * 2u, &tmap_a, &full_bar[st], kx,
                                (int32_t)(wide ? ta * a_rows + TILE_ROWS : p.H + ta * tile_rows));
            };
            auto load_b = [&](uint32_t st, uint32_t kb, uint32_t tb) {
                uint8_t* sb = smem + (size_t)st * stage_bytes + a_bytes;
                const int32_t kx = (int32_t)(kb * BLOCK_K);
                if (GATE && !SWAP) {
                    const uint32_t half = bn / 2u;
                    tma_load_2d(sb, &tmap_b, &full_bar[st], kx, (int32_t)(tb * half));
                    tma_load_2d(sb + half * BLOCK_K * 2u, &tmap_b, &full_bar[st], kx, (int32_t)(p.H + tb * half));
                } else {
                    tma_load_2d(sb, &tmap_b, &full_bar[st], kx, (int32_t)(tb * bn));
                }
            };
            bool first = true;
            for (uint32_t w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
                const uint32_t tile = w / p.splits, z = w - tile * p.splits;
                uint32_t ta, tb;
                tile_coords(p, tile, ta, tb);
                const uint32_t kb0 = z * p.kb_per_split;
                const uint32_t kb1 = (kb0 + p.kb_per_split < p.kblocks) ? kb0 + p.kb_per_split : p.kblocks;
                uint32_t kb = kb0;
                if (first) {
                    // The weights do not depend on the launch ahead of this one: the ring's first
                    // stages take their weight boxes while that launch drains; the activations
                    // follow once it has completed.  (Weights are operand A when swapped, else B.)
                    first = false;
                    const uint32_t npre = (kb1 - kb0 < stages) ? kb1 - kb0 : stages;
                    for (uint32_t i = 0; i < npre; ++i) {        // the ring is empty: no wait needed
                        mbar_expect_tx(&full_bar[i], tx_bytes);
                        if (SWAP) load_a(i, kb0 + i, ta); else load_b(i, kb0 + i, tb);
                    }
                    TC_TRACE(2);
                    dependency_wait();
                    TC_TRACE(3);
                    for (uint32_t i = 0; i < npre; ++i) {
                        if (SWAP) load_b(i, kb0 + i, tb); else load_a(i, kb0 + i, ta);
                    }
                    kb = kb0 + npre;
                    stage = npre == stages ? 0u : npre;
                    phase = npre == stages ? 1u : 0u;
                }
                for (; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(&full_bar[stage], tx_bytes);
                    load_a(stage, kb, ta);
                    load_b(stage, kb, tb);
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (first) dependency_wait();
            TC_TRACE(4);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++iter) {
                const uint32_t tile = w / p.splits, z = w - tile * p.splits;
                const uint32_t kb0 = z * p.kb_per_split;
                const uint32_t kb1 = (kb0 + p.kb_per_split < p.kblocks) ? kb0 + p.kb_per_split : p.kblocks;
                const uint32_t buf = iter % acc_bufs, use = iter / acc_bufs;
                if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * acc_cols;
                for (uint32_t kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    if (iter == 0 && kb == kb0) TC_TRACE(5);
                    const uint32_t sa = smem_u32(smem + (size_t)stage * stage_bytes);
                    const uint32_t sb = sa + a_bytes;
                    const uint64_t a_desc = make_smem_desc(sa);
                    const uint64_t b_desc = make_smem_desc(sb);
#pragma unroll
                    for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
                        // advancing K by 16 elements = 32 bytes inside the swizzled row: +2 in the encoded address
                        umma_f16(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, accum);
                        if (a_boxes == 2u) {
                            const uint64_t a2_desc = make_smem_desc(sa + TILE_ROWS * BLOCK_K * 2u);
                            umma_f16(d_tmem + bn, a2_desc + 2u * k, b_desc + 2u * k, p.idesc, accum);
                        }
                    }
                    umma_commit(&empty_bar[stage]);     // stage reusable once these MMAs retire
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[buf]);     // accumulator complete
                TC_TRACE(6);
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const uint32_t q = warp & 3u;                    // TMEM lane quarter this warp may read
        const uint32_t row_in_tile = q * 32u + lane;
        const uint32_t col_groups = ((blockDim.x >> 5) - 2u) >> 2;   // warps per lane quarter: 1 or 2
        const uint32_t col_group = (warp - 2u) >> 2;                 // this warp's share of the 16-column chunks
        const uint32_t out_cols = GATE ? p.H : p.N;      // width of O
        const uint32_t osz = p.partial ? 4u : dtype_size(p.o_dtype);
        uint32_t iter = 0;
        bool ok = true;
        dependency_wait();      // residuals may come from, and outputs may still be read by, the launch ahead
        for (uint32_t w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++iter) {
            const uint32_t tile = w / p.splits, z = w - tile * p.splits;
            uint32_t ta, tb;
            tile_coords(p, tile, ta, tb);
            const uint32_t buf = iter % acc_bufs, use = iter / acc_bufs;
            if (!mbar_wait(&acc_full[buf], use & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if (threadIdx.x == 64u) TC_TRACE(7);
            const uint32_t t_buf = tmem_base + ((q * 32u) << 16) + buf * acc_cols;
            float bias_n = 0.0f, bias_up = 0.0f;
            if (SWAP && !p.partial && p.bias_mode == OPERAND_PER_COLUMN) {
                const uint32_t n = ta * tile_rows + row_in_tile;
                if (n < out_cols) {
                    bias_n = load_as_f32(p.bias, p.b_dtype, n);
                    if (GATE) bias_up = load_as_f32(p.bias, p.b_dtype, (size_t)p.H + n);
                }
            }
            // columns of the accumulator that map to distinct outputs
            const uint32_t ncols = (GATE && !SWAP) ? bn / 2u : bn;
            // swapped with short weight tiles: lanes past tile_rows belong to the next tile
            const bool row_live = !SWAP || row_in_tile < tile_rows;
            const bool warp_live = !SWAP || q * 32u < tile_rows;
            for (uint32_t sub = 0; sub < (wide ? 2u : 1u); ++sub) {
            const uint32_t t_row = t_buf + sub * bn;                         // second accumulator of a wide tile
            const uint32_t row_base = ta * a_rows + sub * TILE_ROWS;
            for (uint32_t c0 = col_group * 16u; warp_live && c0 < ncols; c0 += 16u * col_groups) {
                uint32_t r0[16], r1[16];
                tmem_ld16(t_row + c0, r0);
                if (GATE) tmem_ld16(t_row + c0 + (SWAP ? bn : bn / 2u), r1);
                tmem_ld_wait();
                if (!SWAP) {
                    store_rows16<GATE>(p, r0, r1, row_base + row_in_tile, tb, c0, z, out_cols, osz);
                } else if (cfold) {
#pragma unroll
                    for (uint32_t c = 0; c < 16u; ++c) red[(c0 + c) * TILE_ROWS + row_in_tile] = __uint_as_float(r0[c]);
                } else if (p.partial) {
                    float* P = p.partial + (size_t)z * p.M * p.N;
                    const uint32_t n = row_base + row_in_tile;
                    const bool row_ok = row_live && (GATE ? (n < p.H) : (n < p.N));
#pragma unroll
                    for (uint32_t c = 0; c < 16u; ++c) {
                        const uint32_t m = tb * bn + c0 + c;
                        if (row_ok && m < p.M) {
                            P[(size_t)m * p.N + n] = __uint_as_float(r0[c]);
                            if (GATE) P[(size_t)m * p.N + p.H + n] = __uint_as_float(r1[c]);
                        }
                    }
                } else {
                    const uint32_t n = row_base + row_in_tile;
                    if (row_live && n < out_cols) {
                        float v[16], u[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) { v[c] = __uint_as_float(r0[c]); u[c] = GATE ? __uint_as_float(r1[c]) : 0.0f; }
                        emit_cols16<GATE>(p, v, u, n, tb * bn + c0, out_cols, bias_n, bias_up);
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (threadIdx.x == 64u) TC_TRACE(8);

            if (p.partial && p.tile_done) {
                // Split-K without a second launch: the CTAs that hold the splits of one tile fold it
                // together.  Each publishes its partial sums and counts itself in; once all `splits`
                // have, each adds up a slice of the tile (every split's partial, in split order, so
                // the result does not depend on who arrived when) and stores the finished outputs.
                // The splits of a tile are neighbouring work items, hence run at the same time on
                // CTAs that are all resident (one per SM): the wait is short, and bounded like every
                // other wait of this kernel.
                const uint32_t fold_parity = iter & 1u;
                __threadfence();                                         // this thread's partials, device-wide
                __syncwarp();
                if (lane == 0) mbar_arrive(fold_in);
                if (threadIdx.x == 64u) {
                    uint32_t go = 0u;
                    if (mbar_wait(fold_in, fold_parity, abort_flag)) {
                        unsigned int* counter = p.tile_done + tile;
                        atomicAdd(counter, 1u);
                        for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
                            unsigned int seen;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                            if (seen >= p.splits) { go = 1u; break; }
                            __nanosleep(64);
                        }
                        if (go) {
                            // counted in a second time once past the wait; the last one through leaves zero behind
                            if (atomicAdd(counter, 1u) == 2u * p.splits - 1u) atomicExch(counter, 0u);
                        } else {
                            *abort_flag = 1u;
                        }
                    }
                    *fold_flag = go;
                    mbar_arrive(fold_out);
                }
                if (!mbar_wait(fold_out, fold_parity, abort_flag)) { ok = false; break; }
                if (!*fold_flag) { ok = false; break; }
                __threadfence();
                {
                    EpilogueArgs ep;
                    ep.bias = p.bias; ep.res = p.res; ep.b_dtype = p.b_dtype; ep.o_dtype = p.o_dtype;
                    ep.has_bias = p.has_bias; ep.has_res = p.has_res; ep.residual_order = p.residual_order;
                    ep.epilogue = p.epilogue; ep.bias_elems = p.bias_elems; ep.res_elems = p.res_elems; ep.scale = p.scale;
                    const size_t MN = (size_t)p.M * p.N;
                    // the axis this CTA takes a slice of: activation rows when swapped (a thread owns an
                    // output column), output columns otherwise (a thread owns an activation row)
                    const uint32_t base = SWAP ? tb * bn : (GATE ? tb * (bn / 2u) : tb * bn);
                    const uint32_t limit = SWAP ? p.M : out_cols;
                    const uint32_t span = SWAP ? bn : ncols;
                    const uint32_t extent = base >= limit ? 0u : (limit - base < span ? limit - base : span);
                    const uint32_t per = (extent + p.splits - 1u) / p.splits;
                    const uint32_t lo = z * per, hi = (lo + per < extent) ? lo + per : extent;
                    for (uint32_t sub = 0; sub < (wide ? 2u : 1u); ++sub) {
                        const uint32_t row = ta * a_rows + sub * TILE_ROWS + row_in_tile;   // swapped: output column; else activation row
                        if (row >= (SWAP ? out_cols : p.M) || !row_live) continue;
                        for (uint32_t i = lo + 4u * col_group; i < hi; i += 4u * col_groups) {
                            float g[4] = {0.0f, 0.0f, 0.0f, 0.0f}, u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            size_t at[4];
#pragma unroll
                            for (uint32_t q = 0; q < 4u; ++q) {
                                const uint32_t j = base + ((i + q < hi) ? i + q : hi - 1u);
                                at[q] = SWAP ? (size_t)j * p.N + row : (size_t)row * p.N + j;
                            }
                            for (uint32_t zz = 0; zz < p.splits; ++zz) {
                                const float* P = p.partial + zz * MN;
#pragma unroll
                                for (uint32_t q = 0; q < 4u; ++q) {
                                    g[q] += __ldcg(P + at[q]);
                                    if (GATE) u[q] += __ldcg(P + at[q] + p.H);
                                }
                            }
#pragma unroll
                            for (uint32_t q = 0; q < 4u; ++q) {
                                if (i + q >= hi) continue;
                                const uint32_t m = SWAP ? base + i + q : row, n = SWAP ? row : base + i + q;
                                const size_t flat = (size_t)m * out_cols + n;
                                const float v = GATE ? finish_gated(ep, g[q], u[q], n, p.H, flat) : finish_output(ep, g[q], flat);
                                store_from_f32(p.O, p.o_dtype, (size_t)m * p.ldo + p.col0 + n, v);
                            }
                        }
                    }
                }
            }
        }
    }

    if (cfold) {
        // The CTAs of the cluster hold the K splits of one tile (split z = rank in the cluster; one work
        // item per CTA).  Every thread of every CTA passes both cluster barriers exactly once, whatever
        // happened before (all waits above are bounded): first "all accumulators are in shared memory",
        // then "nobody reads my shared memory any more".  Between them CTA z adds up columns
        // [z, z + 1) * bn / cfold of all splits, in split order like the fold kernel, and finishes them.
        __syncwarp();
        if (threadIdx.x == 64u) TC_TRACE(10);
        cluster_sync_all();
        if (threadIdx.x == 64u) TC_TRACE(11);
        if (warp >= 2 && !*abort_flag) {
            const uint32_t q = warp & 3u, row_in_tile = q * 32u + lane;
            const uint32_t col_groups = ((blockDim.x >> 5) - 2u) >> 2, col_group = (warp - 2u) >> 2;
            const uint32_t tile = blockIdx.x / p.splits, z = blockIdx.x - tile * p.splits;
            uint32_t ta, tb;
            tile_coords(p, tile, ta, tb);
            const uint32_t n = ta * tile_rows + row_in_tile;
            const uint32_t per = bn / p.cfold;                       // a multiple of 16
            const bool live = row_in_tile < tile_rows && n < p.N;
            const uint32_t red_u32 = smem_u32(red);
            float bias_n = 0.0f;
            if (live && p.bias_mode == OPERAND_PER_COLUMN) bias_n = load_as_f32(p.bias, p.b_dtype, n);
            for (uint32_t k = col_group; k < per / 16u && q * 32u < tile_rows; k += col_groups) {
                const uint32_t c0 = z * per + k * 16u;
                float v[16], u[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) { v[c] = 0.0f; u[c] = 0.0f; }
                for (uint32_t r = 0; r < p.cfold; ++r) {
                    const uint32_t src = map_to_cta(red_u32 + (c0 * TILE_ROWS + row_in_tile) * 4u, r);
#pragma unroll
                    for (uint32_t c = 0; c < 16u; ++c) v[c] += ld_cluster_f32(src + c * TILE_ROWS * 4u);
                }
                if (!live) continue;
                const uint32_t m0 = tb * bn + c0;
                if (p.grp_t1 != kNoGroup) {
                    // a group: plain sums into the member that owns weight row n
                    const uint32_t n1 = p.grp_t1 * TILE_ROWS, n2 = p.grp_t2 == kNoGroup ? p.N : p.grp_t2 * TILE_ROWS;
                    const uint32_t j = n >= n2 ? 2u : (n >= n1 ? 1u : 0u);
                    const uint32_t first = j == 2u ? n2 : (j == 1u ? n1 : 0u);
                    const uint32_t width = (j == 0u ? n1 : (j == 1u ? n2 : p.N)) - first;
#pragma unroll
                    for (uint32_t c = 0; c < 16u; ++c)
                        if (m0 + c < p.M) store_from_f32(p.dst[j], p.o_dtype, (size_t)(m0 + c) * width + (n - first), v[c]);
                } else {
                    emit_cols16<false>(p, v, u, n, m0, p.N, bias_n, 0.0f);
                }
            }
        }
        __syncwarp();
        if (threadIdx.x == 64u) TC_TRACE(12);
        cluster_sync_all();
        if (threadIdx.x == 64u) TC_TRACE(13);
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        atomicExch(p.status, 1);
        // let copies that are still in flight land before the CTA's shared memory is released
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
    if (threadIdx.x == 0) TC_TRACE(9);
}

#ifdef VAICU_TC_TRACE
extern "C" __attribute__((visibility("default"))) int vaicu_debug_tc_trace(unsigned long long* out)
{
    return (int)cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(g_tc_trace));
}
#endif


// ---- CTA-pair variant ------------------------------------------------------
// PTX wrappers for the forms that address the peer CTA of a 2-CTA cluster.
namespace {
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes are counted on an mbarrier of either CTA of the pair
// (every CTA fetches its own boxes; nothing is shared between CTAs by the copy engine).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// One MMA over both CTAs: D[256 x bn] (rows 0-127 in the leader's tensor memory, 128-255
// in the peer's) += A[256 x 16] . B[bn x 16]^T with each CTA holding its 128 rows of A
// and its half of B's rows at the same shared-memory offsets.
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier at this offset in both CTAs once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
}  // namespace

// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x bn tile with
// tcgen05.mma.cta_group::2: each CTA stages its 128 rows of A and HALF of the weights'
// tile, so shared-memory traffic per MMA cycle halves against the single-CTA kernel
// and both accumulator buffers (2 x 256 columns) stay available for overlap.
//   warp 0  (both CTAs) TMA producer for this CTA's boxes; completion bytes of both CTAs
//           are counted on the leader's "full" barrier;
//   warp 1  allocates tensor memory in both CTAs; in the leader (cluster rank 0) one
//           lane issues the MMAs and commits to the barriers of both CTAs;
//   warps 2-5 (both CTAs) epilogue over this CTA's 128 rows; they release an accumulator
//           by arriving on the leader's barrier.
// With GATE the leader's half of B holds the gate rows and the peer's the value rows.
template <bool GATE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads, 1)
tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_b_tail, const __grid_constant__ CUtensorMap tmap_b2, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_ctarank();
    const uint32_t cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const uint32_t bn = p.bn, half = bn / 2u;
    const uint32_t a_bytes = TILE_ROWS * BLOCK_K * 2u;
    const uint32_t b_bytes = half * BLOCK_K * 2u;
    const uint32_t stage_bytes = a_bytes + b_bytes;      // per CTA; multiple of 1024 (bn % 16 == 0)
    const uint32_t stages = p.stages;
    const uint32_t acc_cols = bn;

    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
    uint64_t* empty_bar = full_bar + stages;
    uint64_t* acc_full = empty_bar + stages;      // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2], used in the leader
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // 4 KB per epilogue warp for the staged stores (present when p.staged)
    uint8_t* staging = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tmem_slot + 2) + 127u) & ~(uintptr_t)127u);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (uint32_t b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }   // 4 warps x 2 CTAs
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (p.tail_split > 1u) prefetch_tmap(&tmap_b_tail);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, p.tmem_cols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t num_work = work_items(p);

    // The launch after this one may begin its prologue now (it waits before it touches our results).
    launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            bool first = true;
            for (uint32_t w = cluster_id; w < num_work && ok; w += num_clusters) {
                uint32_t tile, z, strip, bw;
                work_item(p, w, tile, z, strip, bw);
                const uint32_t bh = bw / 2u;                       // rows of B this CTA stages for the item
                uint32_t ta, tb;
                tile_coords(p, tile, ta, tb);
                const uint32_t kb0 = z * p.kb_per_split;
                const uint32_t kb1 = (kb0 + p.kb_per_split < p.kblocks) ? kb0 + p.kb_per_split : p.kblocks;
                const int32_t ya = (int32_t)(ta * 2u * TILE_ROWS + rank * TILE_ROWS);
                int32_t yb = GATE ? (int32_t)((rank ? p.H : 0u) + tb * half + strip * bh) : (int32_t)(tb * bn + strip * bw + rank * bh);
                const CUtensorMap* mb = bw == bn ? &tmap_b : &tmap_b_tail;
                if (!GATE && tb >= p.grp_t1) {
                    // a group: the weight tiles of the second / third member come from their own tensors (the
                    // tail map's slot carries the second member's map; groups run without column strips)
                    const bool third = tb >= p.grp_t2;
                    mb = third ? &tmap_b2 : &tmap_b_tail;
                    yb = (int32_t)((tb - (third ? p.grp_t2 : p.grp_t1)) * bn + rank * bh);
                }
                const uint32_t item_bytes = a_bytes + bh * BLOCK_K * 2u;      // per CTA and k-block
                uint32_t kb = kb0;
                if (first) {
                    // The weights (operand B) do not depend on the launch ahead of this one: the ring's
                    // first stages take their weight boxes while that launch drains; the activations
                    // follow once it has completed.
                    first = false;
                    const uint32_t npre = (kb1 - kb0 < stages) ? kb1 - kb0 : stages;
                    for (uint32_t i = 0; i < npre; ++i) {        // the ring is empty: no wait needed
                        if (rank == 0u) mbar_expect_tx(&full_bar[i], 2u * item_bytes);
                        tma_load_2d_pair(smem + (size_t)i * stage_bytes + a_bytes, mb, map_to_cta(smem_u32(&full_bar[i]), 0u),
                                         (int32_t)((kb0 + i) * BLOCK_K), yb);
                    }
                    dependency_wait();
                    for (uint32_t i = 0; i < npre; ++i)
                        tma_load_2d_pair(smem + (size_t)i * stage_bytes, &tmap_a, map_to_cta(smem_u32(&full_bar[i]), 0u),
                                         (int32_t)((kb0 + i) * BLOCK_K), ya);
                    kb = kb0 + npre;
                    stage = npre == stages ? 0u : npre;
                    phase = npre == stages ? 1u : 0u;
                }
                for (; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    uint8_t* sa = smem + (size_t)stage * stage_bytes;
                    if (rank == 0u) mbar_expect_tx(&full_bar[stage], 2u * item_bytes);   // both CTAs' boxes
                    const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0u);
                    const int32_t kx = (int32_t)(kb * BLOCK_K);
                    tma_load_2d_pair(sa, &tmap_a, bar, kx, ya);
                    tma_load_2d_pair(sa + a_bytes, mb, bar, kx, yb);
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (first) dependency_wait();
            // the leader's last commits land on this CTA's barriers before it may leave
            for (uint32_t s = 0; s < stages && ok; ++s) {
                if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) ok = false;
                if (++stage == stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0u) {
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t w = cluster_id; w < num_work && ok; w += num_clusters, ++iter) {
                uint32_t tile, z, strip, bw;
                work_item(p, w, tile, z, strip, bw);
                const uint32_t idesc = bw == bn ? p.idesc : p.idesc_tail;
                const uint32_t kb0 = z * p.kb_per_split;
                const uint32_t kb1 = (kb0 + p.kb_per_split < p.kblocks) ? kb0 + p.kb_per_split : p.kblocks;
                const uint32_t buf = iter & 1u, use = iter >> 1;
                if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * acc_cols;
                for (uint32_t kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * stage_bytes);
                    const uint64_t a_desc = make_smem_desc(sa);
                    const uint64_t b_desc = make_smem_desc(sa + a_bytes);
#pragma unroll
                    for (uint32_t k = 0; k < BLOCK_K / UMMA_K; ++k)
                        umma_f16_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty_bar[stage]);    // frees the stage in both CTAs
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit_pair(&acc_full[buf]);    // wakes the epilogues of both CTAs
            }
        }
    } else {
        // ---------------- epilogue warps (both CTAs, 128 rows each) ----------------
        const uint32_t q = warp & 3u;
        const uint32_t row_in_tile = q * 32u + lane;
        const uint32_t out_cols = GATE ? p.H : p.N;
        const uint32_t osz = p.partial ? 4u : dtype_size(p.o_dtype);
        uint32_t iter = 0;
        bool ok = true;
        dependency_wait();      // residuals may come from, and outputs may still be read by, the launch ahead
        for (uint32_t w = cluster_id; w < num_work && ok; w += num_clusters, ++iter) {
            uint32_t tile, z, strip, bw;
            work_item(p, w, tile, z, strip, bw);
            const uint32_t bh = bw / 2u;
            const uint32_t ncols = GATE ? bh : bw;                    // output columns of this item
            const uint32_t strip_off = strip * ncols;                 // ... and where they start inside the tile
            uint32_t ta, tb;
            tile_coords(p, tile, ta, tb);
            const uint32_t m = ta * 2u * TILE_ROWS + rank * TILE_ROWS + row_in_tile;
            const uint32_t j_item = (GATE ? tb * half : tb * bn) + strip_off;
            // this row's residual for the item: toward L2 while the accumulator is still being computed,
            // and the first chunk into registers
            const bool res_rows = !p.partial && p.res_mode == OPERAND_FULL && m < p.M;
            if (res_rows) {
                const uint32_t rsz = dtype_size(p.o_dtype);
                const uint8_t* rp = reinterpret_cast<const uint8_t*>(p.res) + ((size_t)m * out_cols + j_item) * rsz;
                const uint32_t span = (j_item + ncols <= out_cols ? ncols : (j_item < out_cols ? out_cols - j_item : 0u)) * rsz;
                for (uint32_t b = 0; b < span; b += 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + b));
            }
            const uint32_t buf = iter & 1u, use = iter >> 1;
            if (!mbar_wait(&acc_full[buf], use & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((q * 32u) << 16) + buf * acc_cols;
            // columns per 128-byte row segment of the output
            const uint32_t seg_cols = 128u / osz;
            ResRaw res_next;
            res_issue(p, m, j_item, out_cols, res_next);
            for (uint32_t c0 = 0; c0 < ncols;) {
                const uint32_t j_seg = j_item + c0;
                const bool stage_it = p.staged && !p.partial && c0 + seg_cols <= ncols && j_seg + seg_cols <= out_cols &&
                                      p.o_aligned16 && (((size_t)p.ldo * osz) % 16u == 0u) && (((size_t)(p.col0 + j_seg) * osz) % 16u == 0u);
                if (!stage_it) {
                    const ResRaw res_cur = res_next;
                    if (c0 + 16u < ncols) res_issue(p, m, j_seg + 16u, out_cols, res_next);      // in flight while this chunk is finished
                    uint32_t r0[16], r1[16];
                    tmem_ld16(t_row + c0, r0);
                    if (GATE) tmem_ld16(t_row + c0 + bh, r1);
                    tmem_ld_wait();
                    store_rows16<GATE>(p, r0, r1, m, tb, strip_off + c0, z, out_cols, osz, &res_cur);
                    c0 += 16u;
                    continue;
                }
                // 1. this thread's row: seg_cols finished values -> its 128-byte line of the warp's staging
                //    block, 16-byte chunks XOR-swizzled by the row so that the 32 lanes hit distinct banks
                uint8_t* mine = staging + (size_t)q * 4096u + (size_t)lane * 128u;
                for (uint32_t g = 0; g < seg_cols; g += 16u) {
                    uint32_t r0[16], r1[16];
                    tmem_ld16(t_row + c0 + g, r0);
                    if (GATE) tmem_ld16(t_row + c0 + g + bh, r1);
                    tmem_ld_wait();
                    float v[16], u[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) { v[c] = __uint_as_float(r0[c]); u[c] = GATE ? __uint_as_float(r1[c]) : 0.0f; }
                    const uint32_t mm = m < p.M ? m : p.M - 1u;          // rows past M compute on a valid row and are not stored
                    finish_row16<GATE>(p, v, u, mm, j_seg + g, out_cols, 16u);
                    if (osz == 4u) {
#pragma unroll
                        for (uint32_t k4 = 0; k4 < 4u; ++k4) {
                            const uint32_t chunk = (g / 4u + k4) ^ (lane & 7u);
                            *reinterpret_cast<float4*>(mine + chunk * 16u) = make_float4(v[4 * k4], v[4 * k4 + 1], v[4 * k4 + 2], v[4 * k4 + 3]);
                        }
                    } else {
#pragma unroll
                        for (uint32_t k8 = 0; k8 < 2u; ++k8) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                if (p.o_dtype == VAICU_DTYPE_F16) {
                                    __half2 h = __floats2half2_rn(v[8 * k8 + 2 * e], v[8 * k8 + 2 * e + 1]);
                                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                                } else {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * k8 + 2 * e], v[8 * k8 + 2 * e + 1]);
                                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                                }
                            }
                            const uint32_t chunk = (g / 8u + k8) ^ (lane & 7u);
                            *reinterpret_cast<uint4*>(mine + chunk * 16u) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
                __syncwarp();
                // 2. eight lanes per row, four rows per store instruction: 4 x 128 contiguous bytes
                const uint32_t m_base = ta * 2u * TILE_ROWS + rank * TILE_ROWS + q * 32u;
#pragma unroll
                for (uint32_t it = 0; it < 8u; ++it) {
                    const uint32_t rr = it * 4u + (lane >> 3), chunk = lane & 7u;
                    const uint4 val = *reinterpret_cast<const uint4*>(staging + (size_t)q * 4096u + (size_t)rr * 128u + ((chunk ^ (rr & 7u)) * 16u));
                    if (m_base + rr < p.M) {
                        uint32_t owner;
                        size_t row;
                        output_row(p, m_base + rr, owner, row);
                        const size_t byte_off = (row * p.ldo + p.col0 + j_seg) * osz + (size_t)chunk * 16u;
                        for (uint32_t d = 0; d < p.n_dst; ++d)
                            if (owner == 0xFFFFFFFFu || d == owner)
                                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.n_dst == 1u ? p.O : p.dst[d]) + byte_off) = val;
                    }
                }
                __syncwarp();
                c0 += seg_cols;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0u));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        atomicExch(p.status, 1);
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves while the other may still signal it or read its tile
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, p.tmem_cols);
    }
}

template <bool GATE>
static cudaError_t launch_pair_variant(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb_tail, const CUtensorMap& mb2,
                                       const TcParams& p, int grid, size_t smem, cudaStream_t stream)
{
    auto kern = tc_gemm_pair_kernel<GATE>;
    static SmemOptIn optin;
    if (cudaError_t e = optin.ensure(kern, (int)kTcMaxSmem); e != cudaSuccess) return e;
    return launch_pdl(kern, dim3((unsigned)grid), dim3(kTcThreads), smem, stream, ma, mb, mb_tail, mb2, p);
}

// CTA-pair kernel over a group of 2-3 weight tensors that share the activations (p.grp_t1 / p.grp_t2: the column
// tile at which the second / third begins; p.dst[0..2] the members' outputs; no column strips in the tail round).
cudaError_t launch_tc_pair_group(const CUtensorMap& map_act, const CUtensorMap* maps_w, const TcParams& p, int grid, size_t smem,
                                 cudaStream_t stream)
{
    return launch_pair_variant<false>(map_act, maps_w[0], maps_w[1], maps_w[2], p, grid, smem, stream);
}

// Number of CTA pairs that can be resident at once (pairs need two SMs of one TPC).
cudaError_t tc_pair_max_clusters(size_t smem, int* clusters)
{
    auto kern = tc_gemm_pair_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcMaxSmem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kTcThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    return cudaOccupancyMaxActiveClusters(clusters, kern, &cfg);
}

// Self-test of the time-out path: one thread waits on an mbarrier that nothing will ever
// arrive on, with a limit of 1024 probes instead of kSpinLimit, and then does exactly what the
// GEMM kernels do when a wait gives up: it records the status word and returns.  No copy is in
// flight, no tensor memory is held, nothing else waits on this thread.
__global__ void __launch_bounds__(32) wait_expiry_selftest_kernel(int* status)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        bool arrived = false;
        for (uint32_t spin = 0; spin < 1024u && !arrived; ++spin) arrived = mbar_try_wait(&bar, 0u);
        if (!arrived) atomicExch(status, 1);
    }
}

cudaError_t launch_wait_expiry_selftest(int* status, cudaStream_t stream)
{
    wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>(status);
    return cudaGetLastError();
}

template <bool SWAP, bool GATE>
static cudaError_t launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ma1, const CUtensorMap& ma2,
                                  const TcParams& p, int grid, size_t smem, cudaStream_t stream)
{
    auto kern = tc_gemm_kernel<SWAP, GATE>;
    static SmemOptIn optin;
    if (cudaError_t e = optin.ensure(kern, (int)kTcMaxSmem); e != cudaSuccess) return e;
    if (SWAP && !GATE && p.cfold)
        return launch_pdl_cluster(kern, dim3((unsigned)grid), dim3(kTcThreadsSwap), smem, stream, p.cfold, ma, mb, ma1, ma2, p);
    return launch_pdl(kern, dim3((unsigned)grid), dim3(SWAP ? kTcThreadsSwap : kTcThreads), smem, stream, ma, mb, ma1, ma2, p);
}

// Clusters of `cluster` CTAs of the swapped kernel that can be resident at once.
cudaError_t tc_swap_max_clusters(size_t smem, unsigned cluster, int* clusters)
{
    auto kern = tc_gemm_kernel<true, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcMaxSmem);
    if (e != cudaSuccess) return e;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1);
    cfg.blockDim = dim3(kTcThreadsSwap, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaOccupancyMaxActiveClusters(clusters, kern, &cfg);
}

// Swapped kernel over a group of 2-3 weight tensors that share the activations (p.grp_t1 / p.grp_t2
// say at which weight tile the second / third begins; p.N is the sum of their rows).
cudaError_t launch_tc_gemm_group(const CUtensorMap* maps_w, const CUtensorMap& map_act, const TcParams& p, int grid, size_t smem,
                                 cudaStream_t stream)
{
    return launch_variant<true, false>(maps_w[0], map_act, maps_w[1], maps_w[2], p, grid, smem, stream);
}

cudaError_t launch_tc_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_b_tail, const TcParams& p,
                           bool swap, int grid, size_t smem, cudaStream_t stream)
{
    const bool gate = p.gate != 0;
    if (p.pair) return gate ? launch_pair_variant<true>(map_a, map_b, map_b_tail, map_b, p, grid, smem, stream)
                            : launch_pair_variant<false>(map_a, map_b, map_b_tail, map_b, p, grid, smem, stream);
    if (swap) return gate ? launch_variant<true, true>(map_a, map_b, map_a, map_a, p, grid, smem, stream)
                          : launch_variant<true, false>(map_a, map_b, map_a, map_a, p, grid, smem, stream);
    return gate ? launch_variant<false, true>(map_a, map_b, map_a, map_a, p, grid, smem, stream)
                : launch_variant<false, false>(map_a, map_b, map_a, map_a, p, grid, smem, stream);
}

}  // namespace vaicu
