// Row-wise argmax over logits [M, N] -> [M] raw uint32 indices: the greedy-decode
// consumer of the lm_head Linear (vAi vai/nodes/argmax.h:9-18, vai/shaders/argmax.comp).
// One block per row, as in the reference; 1024 threads sweep the row with 16-byte loads,
// then (value, index) pairs are folded with warp shuffles.  Ties resolve to the LOWEST
// index (what torch.argmax, the reference's test oracle, returns); NaNs never win.
#include "common.cuh"

namespace vaicu {

namespace {

constexpr int kArgmaxThreads = 1024;

__device__ __forceinline__ void take(float v, uint32_t i, float& best, uint32_t& idx) { argmax_take(v, i, best, idx); }

__global__ void __launch_bounds__(kArgmaxThreads) argmax_kernel(const void* __restrict__ in, int dtype, uint32_t N,
                                                                uint32_t* __restrict__ out)
{
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float best = -3.4028235e38f;        // the shader's start value (argmax.comp:58)
    uint32_t idx = 0u;
    const size_t base = (size_t)row * N;
    if (dtype == VAICU_DTYPE_F32) {
        const float* p = reinterpret_cast<const float*>(in) + base;
        const uint32_t head = (uint32_t)((16u - (reinterpret_cast<uintptr_t>(p) & 15u)) & 15u) / 4u;   // to 16-byte alignment
        const uint32_t h = head < N ? head : N;
        if (tid < h) take(p[tid], tid, best, idx);
        const uint32_t nvec = (N - h) / 4u;
        const float4* pv = reinterpret_cast<const float4*>(p + h);
        for (uint32_t v = tid; v < nvec; v += kArgmaxThreads) {
            const float4 t = pv[v];
            const uint32_t i0 = h + 4u * v;
            take(t.x, i0, best, idx); take(t.y, i0 + 1u, best, idx); take(t.z, i0 + 2u, best, idx); take(t.w, i0 + 3u, best, idx);
        }
        for (uint32_t i = h + 4u * nvec + tid; i < N; i += kArgmaxThreads) take(p[i], i, best, idx);
    } else {
        for (uint32_t i = tid; i < N; i += kArgmaxThreads) take(load_as_f32(in, dtype, base + i), i, best, idx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        take(ov, oi, best, idx);
    }
    __shared__ float s_val[kArgmaxThreads / 32];
    __shared__ uint32_t s_idx[kArgmaxThreads / 32];
    if ((tid & 31u) == 0u) { s_val[tid >> 5] = best; s_idx[tid >> 5] = idx; }
    __syncthreads();
    if (tid < 32u) {
        best = s_val[tid];
        idx = s_idx[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
            take(ov, oi, best, idx);
        }
        if (tid == 0u) out[row] = idx;
    }
}

// Stage 1 of the two-stage form: block (part, row) scans columns [part * seg, (part + 1) * seg)
// of its row (row stride `ld` elements) and writes one (value, index_base + column) pair.
constexpr int kPartThreads = 256;

__global__ void __launch_bounds__(kPartThreads) argmax_part_kernel(const void* __restrict__ in, int dtype, uint32_t N, size_t ld,
                                                                   uint32_t seg, uint32_t index_base, float* __restrict__ out_val,
                                                                   uint32_t* __restrict__ out_idx)
{
    const uint32_t part = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    const uint32_t c0 = part * seg, c1 = (c0 + seg < N) ? c0 + seg : N;
    float best = -3.4028235e38f;
    uint32_t idx = c0;
    const size_t base = (size_t)row * ld;
    if (dtype == VAICU_DTYPE_F32) {
        const float* p = reinterpret_cast<const float*>(in) + base;
        uint32_t c = c0 + tid * 4u;
        const bool vec = ((reinterpret_cast<uintptr_t>(p + c0) & 15u) == 0u);
        if (vec) {
            for (; c + 4u <= c1; c += kPartThreads * 4u) {
                const float4 t = *reinterpret_cast<const float4*>(p + c);
                take(t.x, c, best, idx); take(t.y, c + 1u, best, idx); take(t.z, c + 2u, best, idx); take(t.w, c + 3u, best, idx);
            }
            for (; c < c1; ++c) take(p[c], c, best, idx);      // this thread's ragged tail (at most 3 columns)
        } else {
            for (uint32_t i = c0 + tid; i < c1; i += kPartThreads) take(p[i], i, best, idx);
        }
    } else {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(in) + base;
        uint32_t c = c0 + tid * 8u;
        const bool vec = ((reinterpret_cast<uintptr_t>(p + c0) & 15u) == 0u);
        if (vec) {
            for (; c + 8u <= c1; c += kPartThreads * 8u) {
                const uint4 t = *reinterpret_cast<const uint4*>(p + c);
                const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (uint32_t q = 0; q < 4u; ++q) {
                    float lo, hi;
                    if (dtype == VAICU_DTYPE_F16) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                        lo = f.x; hi = f.y;
                    } else {
                        lo = __uint_as_float(w[q] << 16); hi = __uint_as_float(w[q] & 0xFFFF0000u);
                    }
                    take(lo, c + 2u * q, best, idx);
                    take(hi, c + 2u * q + 1u, best, idx);
                }
            }
            for (; c < c1; ++c) take(load_as_f32(in, dtype, base + c), c, best, idx);
        } else {
            for (uint32_t i = c0 + tid; i < c1; i += kPartThreads) take(load_as_f32(in, dtype, base + i), i, best, idx);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        take(ov, oi, best, idx);
    }
    __shared__ float s_val[kPartThreads / 32];
    __shared__ uint32_t s_idx[kPartThreads / 32];
    if ((tid & 31u) == 0u) { s_val[tid >> 5] = best; s_idx[tid >> 5] = idx; }
    __syncthreads();
    if (tid == 0u) {
        for (int w = 1; w < kPartThreads / 32; ++w) take(s_val[w], s_idx[w], best, idx);
        out_val[(size_t)row * gridDim.x + part] = best;
        out_idx[(size_t)row * gridDim.x + part] = index_base + idx;
    }
}

// Stage 2, and the merge of per-GPU candidates: one warp per row folds `groups` pairs
// found at vals[g * g_stride + row * r_stride]; the lowest index wins among equal values.
__global__ void argmax_merge_kernel(const float* __restrict__ vals, const uint32_t* __restrict__ idxs, uint32_t groups,
                                    size_t g_stride, size_t r_stride, uint32_t M, float* __restrict__ out_val,
                                    uint32_t* __restrict__ out_idx)
{
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (row >= M) return;
    float best = -3.4028235e38f;
    uint32_t idx = 0xFFFFFFFFu;
    for (uint32_t g = lane; g < groups; g += 32u) take(vals[g * g_stride + row * r_stride], idxs[g * g_stride + row * r_stride], best, idx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        take(ov, oi, best, idx);
    }
    if (lane == 0u) {
        if (idx == 0xFFFFFFFFu) idx = idxs[row * r_stride];     // every candidate was NaN or the lowest float: keep the first
        out_idx[row] = idx;
        if (out_val) out_val[row] = best;
    }
}

}  // namespace

cudaError_t launch_argmax(const void* in, int dtype, uint32_t M, uint32_t N, uint32_t* out, cudaStream_t stream)
{
    argmax_kernel<<<M, kArgmaxThreads, 0, stream>>>(in, dtype, N, out);
    return cudaGetLastError();
}

// Column segments per row of the two-stage form: 8192 columns each, at most 256.
uint32_t argmax_parts(uint32_t N)
{
    uint32_t parts = (N + 8191u) / 8192u;
    if (parts > 256u) parts = 256u;
    return parts ? parts : 1u;
}

cudaError_t launch_argmax_pairs(const void* in, int dtype, uint32_t M, uint32_t N, size_t ld, uint32_t index_base, void* workspace,
                                float* out_val, uint32_t* out_idx, cudaStream_t stream)
{
    const uint32_t parts = argmax_parts(N);
    uint32_t seg = (N + parts - 1u) / parts;
    seg = (seg + 7u) & ~7u;                       // segments start on 16-byte boundaries of an aligned row
    float* p_val = reinterpret_cast<float*>(workspace);
    uint32_t* p_idx = reinterpret_cast<uint32_t*>(p_val + (size_t)M * parts);
    argmax_part_kernel<<<dim3(parts, M), kPartThreads, 0, stream>>>(in, dtype, N, ld, seg, index_base, p_val, p_idx);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const uint32_t rows_per_block = 4u;
    argmax_merge_kernel<<<(M + rows_per_block - 1u) / rows_per_block, rows_per_block * 32u, 0, stream>>>(
        p_val, p_idx, parts, 1, parts, M, out_val, out_idx);
    return cudaGetLastError();
}

cudaError_t launch_argmax_merge(const float* vals, const uint32_t* idxs, uint32_t groups, size_t group_stride, uint32_t M,
                                float* out_val, uint32_t* out_idx, cudaStream_t stream)
{
    const uint32_t rows_per_block = 4u;
    argmax_merge_kernel<<<(M + rows_per_block - 1u) / rows_per_block, rows_per_block * 32u, 0, stream>>>(vals, idxs, groups, group_stride, 1,
                                                                                                         M, out_val, out_idx);
    return cudaGetLastError();
}

}  // namespace vaicu
