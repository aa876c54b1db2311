// Row-wise argmax over logits [M, N] -> [M] raw uint32 indices: the greedy-decode
// consumer of the lm_head Linear (vAi vai/nodes/argmax.h:9-18, vai/shaders/argmax.comp).
// One block per row, as in the reference; 1024 threads sweep the row with 16-byte loads,
// then (value, index) pairs are folded with warp shuffles.  Ties resolve to the LOWEST
// index (what torch.argmax, the reference's test oracle, returns); NaNs never win.
#include "common.cuh"

namespace vaicu {

namespace {

constexpr int kArgmaxThreads = 1024;

__device__ __forceinline__ void take(float v, uint32_t i, float& best, uint32_t& idx)
{
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
}

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

}  // namespace

cudaError_t launch_argmax(const void* in, int dtype, uint32_t M, uint32_t N, uint32_t* out, cudaStream_t stream)
{
    argmax_kernel<<<M, kArgmaxThreads, 0, stream>>>(in, dtype, N, out);
    return cudaGetLastError();
}

}  // namespace vaicu
