// CUDA-core kernels of the Linear path:
//   * fma_tile_kernel   — fp32 FFMA tile GEMM.  The only kernel that keeps fp32
//     operands in fp32 end to end (vAi's counterpart is the scalar tile kernel,
//     vai/shaders/linear-tile.comp:68-69,289-295), so fp32 x fp32 layers run
//     here; it also takes every shape the tensor-core kernel cannot (K not a
//     multiple of 8, unaligned views, mixed 16-bit types).
//   * splitk_reduce_kernel — folds split-K partials and applies bias / epilogue /
//     residual / scale (vai/shaders/linear-reduce.comp:88-116), or the fused
//     gate.  Partials are always fp32 here (the reference keeps them in oDtype).
//   * cast_kernel — fp32 activations -> the weights' 16-bit type, the staging the
//     reference's cooperative-matrix kernel does on load
//     (vai/shaders/linear-cm-nv.comp:128-135), as a pre-pass into workspace.
#include "common.cuh"

namespace vaicu {

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TT = 256;

struct FmaParams {
    LinearArgs a;
    float* partial;         // null: write O with the fused epilogue
    uint32_t split_size;    // K span per blockIdx.z
};

__global__ void __launch_bounds__(TT) fma_tile_kernel(const FmaParams p)
{
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    const LinearArgs& a = p.a;
    const uint32_t t = threadIdx.x;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const uint32_t kbeg = blockIdx.z * p.split_size;
    const uint32_t kend = (kbeg + p.split_size < a.K) ? kbeg + p.split_size : a.K;
    const uint32_t lrow = t >> 2, lk = (t & 3u) * 4u;      // loader: 64 rows x 4 k-quads
    const uint32_t ty = t >> 4, tx = t & 15u;              // compute: 16 x 16 threads, 4x4 each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (uint32_t k0 = kbeg; k0 < kend; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t k = k0 + lk + e;
            const bool kin = k < kend;
            const uint32_t m = m0 + lrow, n = n0 + lrow;
            As[lk + e][lrow] = (kin && m < a.M) ? load_as_f32(a.I, a.i_dtype, (size_t)m * a.K + k) : 0.0f;
            Bs[lk + e][lrow] = (kin && n < a.N) ? load_as_f32(a.W, a.w_dtype, (size_t)n * a.K + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float am[4] = {av.x, av.y, av.z, av.w};
            const float bn[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(am[i], bn[j], acc[i][j]);
        }
        __syncthreads();
    }

    const EpilogueArgs ep = make_epilogue_args(a);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = m0 + ty * 4 + i;
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            const size_t flat = (size_t)m * a.N + n;
            if (p.partial) p.partial[(size_t)blockIdx.z * a.M * a.N + flat] = acc[i][j];
            else store_from_f32(a.O, a.o_dtype, flat, finish_output(ep, acc[i][j], flat));
        }
    }
}

struct ReduceParams {
    LinearArgs a;
    const float* partial;
    uint32_t split_count;
};

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const ReduceParams p)
{
    const LinearArgs& a = p.a;
    const EpilogueArgs ep = make_epilogue_args(a);
    const size_t MN = (size_t)a.M * a.N;
    const uint32_t H = a.gate_fuse ? a.N / 2u : a.N;
    const size_t total = (size_t)a.M * H;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        if (!a.gate_fuse) {
            float acc = 0.0f;
            for (uint32_t z = 0; z < p.split_count; ++z) acc += p.partial[z * MN + idx];
            store_from_f32(a.O, a.o_dtype, idx, finish_output(ep, acc, idx));
        } else {
            const uint32_t m = (uint32_t)(idx / H), j = (uint32_t)(idx - (size_t)m * H);
            float g = 0.0f, u = 0.0f;
            for (uint32_t z = 0; z < p.split_count; ++z) {
                g += p.partial[z * MN + (size_t)m * a.N + j];
                u += p.partial[z * MN + (size_t)m * a.N + H + j];
            }
            store_from_f32(a.O, a.o_dtype, idx, finish_gated(ep, g, u, j, H, idx));
        }
    }
}

__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ src, void* __restrict__ dst,
                                                    int dst_dtype, size_t n)
{
    const size_t nvec = n / 8u;
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, gstride = (size_t)gridDim.x * blockDim.x;
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (aligned) {
        for (size_t v = gid; v < nvec; v += gstride) {
            const float4 a = reinterpret_cast<const float4*>(src)[2 * v];
            const float4 b = reinterpret_cast<const float4*>(src)[2 * v + 1];
            uint4 o;
            if (dst_dtype == VAICU_DTYPE_F16) {
                __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
                __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
                o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
            } else {
                __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
                o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
            }
            reinterpret_cast<uint4*>(dst)[v] = o;
        }
        for (size_t i = nvec * 8u + gid; i < n; i += gstride) store_from_f32(dst, dst_dtype, i, src[i]);
    } else {
        for (size_t i = gid; i < n; i += gstride) store_from_f32(dst, dst_dtype, i, src[i]);
    }
}

}  // namespace

cudaError_t launch_fma_tile(const LinearArgs& a, const FmaTileConfig& cfg, float* partial, cudaStream_t stream)
{
    FmaParams p{};
    p.a = a;
    p.partial = partial;
    p.split_size = cfg.split_size;
    dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM, cfg.split_count);
    if (grid.y > 65535u || grid.z > 65535u) return cudaErrorInvalidConfiguration;
    fma_tile_kernel<<<grid, TT, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_splitk_reduce(const LinearArgs& a, const float* partial, uint32_t split_count, cudaStream_t stream)
{
    ReduceParams p{};
    p.a = a;
    p.partial = partial;
    p.split_count = split_count;
    const size_t total = (size_t)a.M * (a.gate_fuse ? a.N / 2u : a.N);
    size_t blocks = (total + 255u) / 256u;
    if (blocks > 148u * 16u) blocks = 148u * 16u;
    if (blocks == 0) blocks = 1;
    splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_cast_f32_to_16(const float* src, void* dst, int dst_dtype, size_t n, int sm_count, cudaStream_t stream)
{
    size_t blocks = (n / 8u + 255u) / 256u;
    const size_t cap = (size_t)sm_count * 8u;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    cast_kernel<<<(unsigned)blocks, 256, 0, stream>>>(src, dst, dst_dtype, n);
    return cudaGetLastError();
}

}  // namespace vaicu
