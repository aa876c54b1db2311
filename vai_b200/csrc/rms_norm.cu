// Row normalisations over the feature axis, the producers of a Linear's activations.
// RmsNorm, Llama / Gemma blocks (vAi vai/nodes/rms-norm.h:9-24, vai/shaders/rms-norm.comp):
//   O[i, j] = I[i, j] * rsqrt(mean(I[i, :]^2) + eps) (* scale[j]) (+ shift[j]) (+ R[i, j])
// LayerNorm, GPT-2 blocks (vAi vai/nodes/layer-norm.h:9-31, vai/shaders/layer-norm.comp):
//   O[i, j] = (I[i, j] - mean_i) * rsqrt(var_i + eps) * scale[j] (+ shift[j]) (+ R[i, j])
//   with the reference's shifted one-pass statistics (s = I[i, 0]; sums of (x - s) and
//   (x - s)^2; mean = s + sum / F; var = max(sumSq - sum^2 / F, 0) / F).
// One block per row; the row is read once into registers (up to 16 values per thread,
// beyond that it is re-read), the sum of squares is accumulated in fp32 whatever the
// I/O dtypes, and the output is written in the dtype the consumer wants — 16-bit output
// feeds the tensor-core Linear directly, without the cast pre-pass.
#include "common.cuh"

namespace vaicu {

namespace {

constexpr int kRmsThreads = 256;
constexpr int kRmsCache = 16;    // values a thread keeps in registers: rows up to 4096 are read once

struct RmsParams {
    const void* in;
    const void* scale;
    const void* shift;
    const void* res;
    void* out;
    uint32_t rows, feat;
    int32_t i_dtype, w_dtype, o_dtype;
    float eps;
};

template <bool LAYER>
__global__ void __launch_bounds__(kRmsThreads) row_norm_kernel(const RmsParams p)
{
    const uint32_t tid = threadIdx.x;
    __shared__ float s_part[kRmsThreads / 32];
    __shared__ float s_part2[kRmsThreads / 32];
    __shared__ float s_inv, s_mean;
    for (uint32_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const size_t base = (size_t)row * p.feat;
        float cache[kRmsCache];
        float sq = 0.0f, sum = 0.0f;
        const float sh = LAYER ? load_as_f32(p.in, p.i_dtype, base) : 0.0f;
#pragma unroll
        for (int c = 0; c < kRmsCache; ++c) {
            const uint32_t j = tid + (uint32_t)c * kRmsThreads;
            cache[c] = j < p.feat ? load_as_f32(p.in, p.i_dtype, base + j) : sh;
            const float d = cache[c] - sh;
            sq += d * d;
            if (LAYER) sum += d;
        }
        for (uint32_t j = tid + kRmsCache * kRmsThreads; j < p.feat; j += kRmsThreads) {
            const float d = load_as_f32(p.in, p.i_dtype, base + j) - sh;
            sq += d * d;
            if (LAYER) sum += d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
            if (LAYER) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        }
        if ((tid & 31u) == 0u) { s_part[tid >> 5] = sq; if (LAYER) s_part2[tid >> 5] = sum; }
        __syncthreads();
        if (tid == 0u) {
            float q = 0.0f, s = 0.0f;
            for (int w = 0; w < kRmsThreads / 32; ++w) { q += s_part[w]; if (LAYER) s += s_part2[w]; }
            if (LAYER) {
                const float m2 = fmaxf(q - s * s / (float)p.feat, 0.0f);       // layer-norm.comp:183-186
                s_mean = sh + s / (float)p.feat;
                s_inv = rsqrtf(m2 / (float)p.feat + p.eps);
            } else {
                s_mean = 0.0f;
                s_inv = rsqrtf(q / (float)p.feat + p.eps);     // inversesqrt(mean + eps), rms-norm.comp
            }
        }
        __syncthreads();
        const float inv = s_inv, mean = s_mean;
        auto finish = [&](uint32_t j, float x) {
            float v = LAYER ? (x - mean) * inv : x * inv;
            if (p.scale) v *= load_as_f32(p.scale, p.w_dtype, j);
            if (p.shift) v += load_as_f32(p.shift, p.w_dtype, j);
            if (p.res) v += load_as_f32(p.res, p.i_dtype, base + j);
            store_from_f32(p.out, p.o_dtype, base + j, v);
        };
#pragma unroll
        for (int c = 0; c < kRmsCache; ++c) {
            const uint32_t j = tid + (uint32_t)c * kRmsThreads;
            if (j < p.feat) finish(j, cache[c]);
        }
        for (uint32_t j = tid + kRmsCache * kRmsThreads; j < p.feat; j += kRmsThreads)
            finish(j, load_as_f32(p.in, p.i_dtype, base + j));
        __syncthreads();     // s_part / s_inv are reused by the next row
    }
}

}  // namespace

cudaError_t launch_rms_norm(const void* in, const void* scale, const void* shift, const void* res, void* out, uint32_t rows,
                            uint32_t feat, int i_dtype, int w_dtype, int o_dtype, float eps, int sm_count, cudaStream_t stream)
{
    RmsParams p{in, scale, shift, res, out, rows, feat, i_dtype, w_dtype, o_dtype, eps};
    uint32_t grid = rows;
    const uint32_t cap = (uint32_t)sm_count * 8u;
    if (grid > cap) grid = cap;
    row_norm_kernel<false><<<grid, kRmsThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_layer_norm(const void* in, const void* scale, const void* shift, const void* res, void* out, uint32_t rows,
                              uint32_t feat, int i_dtype, int w_dtype, int o_dtype, float eps, int sm_count, cudaStream_t stream)
{
    RmsParams p{in, scale, shift, res, out, rows, feat, i_dtype, w_dtype, o_dtype, eps};
    uint32_t grid = rows;
    const uint32_t cap = (uint32_t)sm_count * 8u;
    if (grid > cap) grid = cap;
    row_norm_kernel<true><<<grid, kRmsThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace vaicu
