// GatedMul as a kernel of its own: O[r, j] = act(I[r, j]) * I[r, H + j] over rows of 2H
// elements (vAi vai/nodes/gated-mul.h:9-20, vai/shaders/gated-mul.comp:38-49).
//
// A gate|value Linear followed by this node is normally recorded as ONE launch (the
// Linear kernels apply the gate in their epilogue); this kernel is what runs when the
// pair cannot be fused: the Linear's output has a second reader, the Linear carries an
// epilogue, a scale or a residual of its own, or the node stands alone.
//
// Pure streaming: 2H values in, H out per row.  Each thread takes 16 bytes of the gate
// half and the 16 bytes at the same offset of the value half, so a warp reads two
// contiguous 512-byte runs per step; rows that do not allow 16-byte steps (H not a
// multiple of the vector width, or a base that is not 16-byte aligned) go element by
// element.  The activation is the exact-constant fp32 form the reference's shader uses
// (vai/shaders/common/activation.h:19-58), not the fast-math one of the GEMM epilogue.
#include "common.cuh"

namespace vaicu {

namespace {

template <int ISZ> struct InVec;
template <> struct InVec<4> { static constexpr int N = 4; };   // 4 fp32 per 16 bytes
template <> struct InVec<2> { static constexpr int N = 8; };   // 8 fp16 / bf16 per 16 bytes

// N consecutive elements starting at `idx` (16-byte aligned) widened to fp32.
template <int ISZ>
__device__ __forceinline__ void load_vec(const void* base, int dt, size_t idx, float* f)
{
    if (ISZ == 4) {
        const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
        f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w;
    } else {
        const uint4 t = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (dt == VAICU_DTYPE_F16) {
                const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                f[2 * q] = p.x; f[2 * q + 1] = p.y;
            } else {
                f[2 * q] = __uint_as_float(w[q] << 16);
                f[2 * q + 1] = __uint_as_float(w[q] & 0xFFFF0000u);
            }
        }
    }
}

// V finished values -> O[idx ..], as 8-, 16- or 32-byte stores when the base allows it.
template <int V>
__device__ __forceinline__ void store_vec(void* out, int o_dtype, size_t idx, const float* v, bool out_aligned16)
{
    if (!out_aligned16) {
#pragma unroll
        for (int c = 0; c < V; ++c) store_from_f32(out, o_dtype, idx + c, v[c]);
        return;
    }
    if (o_dtype == VAICU_DTYPE_F32) {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + idx);
#pragma unroll
        for (int q = 0; q < V / 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        return;
    }
    uint32_t w[V / 2];
#pragma unroll
    for (int q = 0; q < V / 2; ++q) {
        if (o_dtype == VAICU_DTYPE_F16) {
            __half2 h = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
            w[q] = *reinterpret_cast<uint32_t*>(&h);
        } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
            w[q] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    uint16_t* dst = reinterpret_cast<uint16_t*>(out) + idx;
    if (V == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2 % (V / 2)], w[3 % (V / 2)]);
    else *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
}

template <int ISZ>
__global__ void __launch_bounds__(256) gated_mul_vec_kernel(const void* __restrict__ in, void* __restrict__ out, uint32_t rows,
                                                            uint32_t H, int i_dtype, int o_dtype, int act)
{
    constexpr int V = InVec<ISZ>::N;
    const bool out_aligned16 = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    const uint32_t per_row = H / V;
    const size_t total = (size_t)rows * per_row;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(v / per_row), j = (uint32_t)(v - (size_t)r * per_row) * V;
        float g[V], u[V];
        load_vec<ISZ>(in, i_dtype, (size_t)r * 2u * H + j, g);
        load_vec<ISZ>(in, i_dtype, (size_t)r * 2u * H + H + j, u);
#pragma unroll
        for (int c = 0; c < V; ++c) g[c] = apply_epilogue(act, g[c]) * u[c];
        store_vec<V>(out, o_dtype, (size_t)r * H + j, g, out_aligned16);
    }
}

__global__ void __launch_bounds__(256) gated_mul_scalar_kernel(const void* __restrict__ in, void* __restrict__ out, uint32_t rows,
                                                               uint32_t H, int i_dtype, int o_dtype, int act)
{
    const size_t total = (size_t)rows * H;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / H, src = r * 2u * H + (e - r * H);      // gated-mul.comp:45-46
        store_from_f32(out, o_dtype, e, apply_epilogue(act, load_as_f32(in, i_dtype, src)) * load_as_f32(in, i_dtype, src + H));
    }
}

}  // namespace

cudaError_t launch_gated_mul(const void* in, void* out, uint32_t rows, uint32_t H, int i_dtype, int o_dtype, int act,
                             int sm_count, cudaStream_t stream)
{
    const uint32_t isz = dtype_size(i_dtype);
    const uint32_t vec = 16u / isz;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) & 15u) == 0) && (H % vec == 0u);
    const size_t work = aligned ? (size_t)rows * (H / vec) : (size_t)rows * H;
    size_t blocks = (work + 255u) / 256u;
    const size_t cap = (size_t)(sm_count > 0 ? sm_count : 148) * 8u;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    if (!aligned) gated_mul_scalar_kernel<<<(unsigned)blocks, 256, 0, stream>>>(in, out, rows, H, i_dtype, o_dtype, act);
    else if (isz == 4u) gated_mul_vec_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(in, out, rows, H, i_dtype, o_dtype, act);
    else gated_mul_vec_kernel<2><<<(unsigned)blocks, 256, 0, stream>>>(in, out, rows, H, i_dtype, o_dtype, act);
    return cudaGetLastError();
}

}  // namespace vaicu
