// Row-wise top-k sampling over logits [M, N]: vAi's TopKSampling node
// (vai/nodes/topk-sampling.h:9-31, vai/shaders/topk-sampling.comp):
//   out[i] = sample(softmax(top-k(I[i, :]) / temperature), u)
// with the reference's exact rules: candidates ranked by (value descending, index
// ascending); Z and the running sum accumulated in that order in fp32 with the row maximum
// subtracted; the first rank whose running sum reaches u * Z is the sample (rank 0 if none).
//
// Two launches, as in the reference.  Stage 1: block (g, row) keeps its 2048-column slice in
// registers (8 per thread, each thread's list sorted descending), then k rounds of a block-wide
// "best head" reduction pop the slice's top-k in order.  Stage 2: one block per row does the
// same over the G * k candidates and thread 0 samples.  Rows of at most 8192 columns need
// stage 2 only.  u lives in device memory so that a recorded launch sees each step's value.
#include "common.cuh"

namespace vaicu {

namespace {

constexpr uint32_t kList = 8;             // register list length per thread
constexpr uint32_t kMaxK = 128;           // vAi TopKSampling::maxK
constexpr uint32_t kPartThreads = 256;    // stage 1: 256 * 8 = 2048 columns per block
constexpr uint32_t kSlice = kPartThreads * kList;
constexpr float kLowest = -3.4028235e38f; // the shader's sentinel (finite: softmax terms stay NaN-free)

__device__ __forceinline__ bool outranks(float av, uint32_t ai, float bv, uint32_t bi)
{
    return av > bv || (av == bv && ai < bi);
}

struct TopkParams {
    const void* logits;       // stage 1 / single stage: [M, N] of dtype
    const uint2* cand_in;     // stage 2: [M, n_in] (value bits, index)
    uint2* cand_out;          // stage 1: [M, G * k]
    uint32_t* out;            // final stage: [M]
    const float* u;           // device scalar in [0, 1)
    uint32_t N;               // elements per row this launch reads
    uint32_t k;               // min(K, row width of the logits)
    int32_t dtype;
    float temperature;
};

// FINAL: this launch samples (reads logits when cand_in is null, else candidates).
template <bool FINAL>
__global__ void topk_kernel(const TopkParams p)
{
    const uint32_t row = blockIdx.y, g = blockIdx.x, G = gridDim.x, tid = threadIdx.x, nthreads = blockDim.x;
    __shared__ float s_val[32];
    __shared__ uint32_t s_idx[32];
    __shared__ float top_v[kMaxK];
    __shared__ uint32_t top_i[kMaxK];

    float lv[kList];
    uint32_t li[kList];
#pragma unroll
    for (uint32_t j = 0; j < kList; ++j) { lv[j] = kLowest; li[j] = 0xFFFFFFFFu; }

    const uint32_t slice = (p.N + G - 1u) / G;
    const uint32_t s0 = g * slice, s1 = (s0 + slice < p.N) ? s0 + slice : p.N;
    for (uint32_t i = s0 + tid; i < s1; i += nthreads) {
        float v;
        uint32_t idx;
        if (p.cand_in) {
            const uint2 c = p.cand_in[(size_t)row * p.N + i];
            v = __uint_as_float(c.x);
            idx = c.y;
        } else {
            v = load_as_f32(p.logits, p.dtype, (size_t)row * p.N + i);
            idx = i;
        }
        // insertion into the descending list (fully unrolled: the list stays in registers)
        if (outranks(v, idx, lv[kList - 1], li[kList - 1])) {
            lv[kList - 1] = v; li[kList - 1] = idx;
#pragma unroll
            for (int q = kList - 1; q > 0; --q) {
                if (outranks(lv[q], li[q], lv[q - 1], li[q - 1])) {
                    const float tv = lv[q]; lv[q] = lv[q - 1]; lv[q - 1] = tv;
                    const uint32_t ti = li[q]; li[q] = li[q - 1]; li[q - 1] = ti;
                }
            }
        }
    }

    // k rounds: the best list head of the block wins the round and its thread pops
    const uint32_t nwarps = nthreads >> 5;
    for (uint32_t r = 0; r < p.k; ++r) {
        float bv = lv[0];
        uint32_t bi = li[0];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (outranks(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31u) == 0u) { s_val[tid >> 5] = bv; s_idx[tid >> 5] = bi; }
        __syncthreads();
        bv = s_val[0]; bi = s_idx[0];
        for (uint32_t w = 1; w < nwarps; ++w)
            if (outranks(s_val[w], s_idx[w], bv, bi)) { bv = s_val[w]; bi = s_idx[w]; }
        if (tid == 0u) { top_v[r] = bv; top_i[r] = bi; }
        if (lv[0] == bv && li[0] == bi) {          // this thread's head won: advance its list
#pragma unroll
            for (uint32_t q = 0; q + 1u < kList; ++q) { lv[q] = lv[q + 1]; li[q] = li[q + 1]; }
            lv[kList - 1] = kLowest; li[kList - 1] = 0xFFFFFFFFu;
        }
        __syncthreads();
    }

    if (!FINAL) {
        if (tid < p.k) p.cand_out[((size_t)row * G + g) * p.k + tid] = make_uint2(__float_as_uint(top_v[tid]), top_i[tid]);
        return;
    }
    if (tid == 0u) {
        // temperature softmax over the k winners and the inverse-CDF sample (topk-sampling.comp:237-258)
        const float inv_t = 1.0f / fmaxf(p.temperature, 1e-6f);
        const float m = top_v[0];
        float z = 0.0f;
        for (uint32_t r = 0; r < p.k; ++r) z += expf((top_v[r] - m) * inv_t);
        const float target = *p.u * z;
        float cum = 0.0f;
        uint32_t chosen = top_i[0];
        for (uint32_t r = 0; r < p.k; ++r) {
            cum += expf((top_v[r] - m) * inv_t);
            if (cum >= target) { chosen = top_i[r]; break; }
        }
        p.out[row] = chosen;
    }
}

uint32_t final_threads(uint32_t n)
{
    uint32_t t = ((n + kList - 1u) / kList + 31u) / 32u * 32u;
    if (t < 32u) t = 32u;
    return t > 1024u ? 1024u : t;
}

}  // namespace

// Blocks per row in stage 1 (1: single launch).
uint32_t topk_groups(uint32_t N) { return N <= 1024u * kList ? 1u : (N + kSlice - 1u) / kSlice; }

cudaError_t launch_topk_sample(const void* logits, int dtype, uint32_t M, uint32_t N, uint32_t K, float temperature,
                               const float* u, void* workspace, uint32_t* out, cudaStream_t stream)
{
    TopkParams p{};
    p.logits = logits; p.dtype = dtype; p.temperature = temperature; p.u = u; p.out = out;
    p.k = K < N ? K : N;
    const uint32_t G = topk_groups(N);
    if (G == 1u) {
        p.N = N;
        topk_kernel<true><<<dim3(1, M), final_threads(N), 0, stream>>>(p);
        return cudaGetLastError();
    }
    p.N = N;
    p.cand_out = reinterpret_cast<uint2*>(workspace);
    topk_kernel<false><<<dim3(G, M), kPartThreads, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    TopkParams q = p;
    q.logits = nullptr;
    q.cand_in = reinterpret_cast<const uint2*>(workspace);
    q.cand_out = nullptr;
    q.N = G * p.k;
    topk_kernel<true><<<dim3(1, M), final_threads(q.N), 0, stream>>>(q);
    return cudaGetLastError();
}

}  // namespace vaicu
