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
#include <mutex>

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

    // Four consecutive k of one row of each operand per thread, held in registers for one trip:
    // the loads of trip i + 1 are in flight while trip i is multiplied out of shared memory.
    const uint32_t lm = m0 + lrow, ln = n0 + lrow;
    const bool quad_i = a.i_dtype == VAICU_DTYPE_F32 && a.K % 4u == 0 && kbeg % 4u == 0 && (reinterpret_cast<uintptr_t>(a.I) & 15u) == 0;
    const bool quad_w = a.w_dtype == VAICU_DTYPE_F32 && a.K % 4u == 0 && kbeg % 4u == 0 && (reinterpret_cast<uintptr_t>(a.W) & 15u) == 0;
    float ra[4], rb[4];
    auto fetch = [&](uint32_t k0) {
        const uint32_t k = k0 + lk;
        if (quad_i && lm < a.M && k + 3u < kend) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.I) + (size_t)lm * a.K + k));
            ra[0] = v.x; ra[1] = v.y; ra[2] = v.z; ra[3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) ra[e] = (k + e < kend && lm < a.M) ? load_as_f32(a.I, a.i_dtype, (size_t)lm * a.K + k + e) : 0.0f;
        }
        if (quad_w && ln < a.N && k + 3u < kend) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.W) + (size_t)ln * a.K + k));
            rb[0] = v.x; rb[1] = v.y; rb[2] = v.z; rb[3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) rb[e] = (k + e < kend && ln < a.N) ? load_as_f32(a.W, a.w_dtype, (size_t)ln * a.K + k + e) : 0.0f;
        }
    };
    if (kbeg < kend) fetch(kbeg);
    for (uint32_t k0 = kbeg; k0 < kend; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            As[lk + e][lrow] = ra[e];
            Bs[lk + e][lrow] = rb[e];
        }
        __syncthreads();
        if (k0 + BK < kend) fetch(k0 + BK);
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
    launch_dependents();
    dependency_wait();          // the partial sums come from the launch ahead of this one
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

// Fold of a group's split-K partials (q / k / v computed as one swapped tensor-core launch): the partial
// sums are [splits][M][N] over the members' rows side by side; the members' outputs are separate
// dense tensors.  Four columns per thread: members are multiples of 128 rows, so a quad never straddles two.
struct GroupFoldParams {
    const float* partial;
    uint32_t splits, M, N, count;
    uint32_t start[4];          // first column of member i; start[count] = N
    void* O[3];
    int o_dtype;
};

__global__ void __launch_bounds__(256) group_fold_kernel(const GroupFoldParams p)
{
    launch_dependents();
    dependency_wait();          // the partial sums come from the launch ahead of this one
    const size_t MN = (size_t)p.M * p.N;
    const uint32_t quads_per_row = p.N / 4u;
    const size_t total = (size_t)p.M * quads_per_row;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const uint32_t m = (uint32_t)(idx / quads_per_row);
        const uint32_t n = (uint32_t)(idx - (size_t)m * quads_per_row) * 4u;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float* src = p.partial + (size_t)m * p.N + n;
        for (uint32_t z = 0; z < p.splits; ++z) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + z * MN));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        uint32_t j = 0;
        if (p.count > 2u && n >= p.start[2]) j = 2u;
        else if (n >= p.start[1]) j = 1u;
        const uint32_t width = p.start[j + 1u] - p.start[j];
        const size_t at = (size_t)m * width + (n - p.start[j]);
        if (p.o_dtype == VAICU_DTYPE_F32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.O[j]) + at) = acc;
        } else {
            uint2 o;
            if (p.o_dtype == VAICU_DTYPE_F16) {
                __half2 h0 = __floats2half2_rn(acc.x, acc.y), h1 = __floats2half2_rn(acc.z, acc.w);
                o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
            } else {
                __nv_bfloat162 h0 = __floats2bfloat162_rn(acc.x, acc.y), h1 = __floats2bfloat162_rn(acc.z, acc.w);
                o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
            }
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.O[j]) + at) = o;
        }
    }
}

__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ src, void* __restrict__ dst,
                                                    int dst_dtype, size_t n)
{
    launch_dependents();
    dependency_wait();          // the activations come from the launch ahead of this one
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

cudaError_t launch_group_fold(const float* partial, uint32_t splits, uint32_t M, uint32_t count, const uint32_t* rows,
                              void* const* O, int o_dtype, cudaStream_t stream)
{
    GroupFoldParams p{};
    p.partial = partial; p.splits = splits; p.M = M; p.count = count; p.o_dtype = o_dtype;
    uint32_t at = 0;
    for (uint32_t i = 0; i < count; ++i) { p.start[i] = at; p.O[i] = O[i]; at += rows[i]; }
    for (uint32_t i = count; i < 4u; ++i) p.start[i] = at;
    p.N = at;
    const size_t total = (size_t)M * (at / 4u);
    size_t blocks = (total + 255u) / 256u;
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    if (blocks == 0) blocks = 1;
    return launch_pdl(group_fold_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, p);
}

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
    return launch_pdl(splitk_reduce_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, p);
}

cudaError_t launch_cast_f32_to_16(const float* src, void* dst, int dst_dtype, size_t n, int sm_count, cudaStream_t stream)
{
    size_t blocks = (n / 8u + 255u) / 256u;
    const size_t cap = (size_t)sm_count * 8u;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return launch_pdl(cast_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, src, dst, dst_dtype, n);
}


// ---------------------------------------------------------------------------
// Split-K Linear for hosts that may not allocate.
//
// Some embedders own every byte of device memory themselves — a serving process
// that pre-partitions the heap at start-up and forbids allocation afterwards, or a
// plugin host whose sandbox exposes no allocator — so they can hand over the
// operands they already hold but have no way to obtain the `workspace` that
// vaicu_linear_run() wants for split-K partial sums.  For them the partial sums
// live in the fixed array below, which is part of the library image: every GPU
// that loads the library carries these 8 MiB until the process exits.
//
// The array's name is only meaningful to device code and to cudaGetSymbolAddress;
// host code must never pass `g_splitk_scratch` itself to a kernel.  The address is
// looked up once per device (with that device current) and cached.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB: split_count * M * N fp32 partials must fit
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_splitk_scratch[kStaticScratchBytes];

std::mutex g_scratch_mutex;
void* g_scratch_addr[kMaxDevices] = {};
int g_scratch_sms[kMaxDevices] = {};

// Device address of the scratch array on the current device; looked up on the first
// call per device.  Returns a status code.
int static_scratch_for_current_device(float** out, int* sm_count)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_last_error("cudaGetDevice", cudaGetErrorString(e)); return VAICU_ERR_CUDA; }
    if (dev < 0 || dev >= kMaxDevices) { set_last_error("vaicu_linear_splitk_static", "device ordinal out of range"); return VAICU_ERR_INVALID_VALUE; }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_splitk_scratch);
        if (e != cudaSuccess || !ptr) {
            set_last_error("cudaGetSymbolAddress(g_splitk_scratch)", cudaGetErrorString(e));
            (void)cudaGetLastError();
            return VAICU_ERR_CUDA;
        }
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) { set_last_error("cudaDeviceGetAttribute", cudaGetErrorString(e)); return VAICU_ERR_CUDA; }
        g_scratch_sms[dev] = sms;
        g_scratch_addr[dev] = ptr;
    }
    *out = reinterpret_cast<float*>(g_scratch_addr[dev]);
    *sm_count = g_scratch_sms[dev];
    return VAICU_OK;
}

}  // namespace
}  // namespace vaicu

#pragma GCC visibility push(default)
extern "C" int vaicu_linear_splitk_static(const vaicu_linear_desc* d, vaicu_stream_t stream, const void* I, const void* W,
                                          const void* bias, const void* residual, void* O)
{
    using namespace vaicu;
    if (!d || !I || !W || !O) return VAICU_ERR_INVALID_VALUE;
    if (d->M == 0 || d->N == 0 || d->K == 0) return VAICU_ERR_INVALID_VALUE;
    auto ok_dtype = [](int t) { return t == VAICU_DTYPE_F32 || t == VAICU_DTYPE_F16 || t == VAICU_DTYPE_BF16; };
    if (!ok_dtype(d->i_dtype) || !ok_dtype(d->w_dtype) || !ok_dtype(d->o_dtype)) return VAICU_ERR_INVALID_VALUE;
    if (d->has_bias && (!ok_dtype(d->b_dtype) || !bias)) return VAICU_ERR_INVALID_VALUE;
    if (d->has_residual && !residual) return VAICU_ERR_INVALID_VALUE;
    if (d->epilogue < 0 || d->epilogue > VAICU_EPILOGUE_SIGMOID) return VAICU_ERR_INVALID_VALUE;
    if (d->residual_order != 0 && d->residual_order != 1) return VAICU_ERR_INVALID_VALUE;
    if (d->split_size != 0 && d->split_size < 32) return VAICU_ERR_INVALID_VALUE;
    if (d->gate_fuse) return VAICU_ERR_UNSUPPORTED;
    if ((uint64_t)d->M * d->N >= (1ull << 32)) return VAICU_ERR_INVALID_VALUE;
    if (d->has_bias && d->bias_elems && (d->bias_elems % d->N || ((uint64_t)d->M * d->N) % d->bias_elems)) return VAICU_ERR_INVALID_VALUE;
    if (d->has_residual && d->residual_elems && (d->residual_elems % d->N || ((uint64_t)d->M * d->N) % d->residual_elems))
        return VAICU_ERR_INVALID_VALUE;
    // Same rule as vaicu_linear_run: every operand aligned to its element size.  Checked before
    // anything touches the GPU, so a bad pointer comes back as a status instead of a
    // misaligned-address fault inside the kernel.
    auto elem_aligned = [](const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dtype_size(dt) - 1u)) == 0; };
    if (!elem_aligned(I, d->i_dtype) || !elem_aligned(W, d->w_dtype) || !elem_aligned(O, d->o_dtype)) return VAICU_ERR_ALIGNMENT;
    if (d->has_bias && !elem_aligned(bias, d->b_dtype)) return VAICU_ERR_ALIGNMENT;
    if (d->has_residual && !elem_aligned(residual, d->o_dtype)) return VAICU_ERR_ALIGNMENT;

    float* scratch = nullptr;
    int sms = 0;
    const int rc = static_scratch_for_current_device(&scratch, &sms);
    if (rc != VAICU_OK) return rc;

    // K spans: the caller's split_size, else enough spans to occupy the SMs
    FmaTileConfig cfg;
    cfg.split_size = d->K;
    cfg.split_count = 1;
    if (d->split_size) {
        cfg.split_size = d->split_size < d->K ? d->split_size : d->K;
    } else {
        const uint32_t tiles = ((d->M + 63u) / 64u) * ((d->N + 63u) / 64u);
        if (tiles * 2u <= (uint32_t)sms && d->K >= 1024u) {
            uint32_t want = (uint32_t)sms / tiles;
            if (want > 16u) want = 16u;
            cfg.split_size = ((d->K + want - 1u) / want + 63u) / 64u * 64u;
        }
    }
    cfg.split_count = (d->K + cfg.split_size - 1u) / cfg.split_size;
    const uint64_t need = (uint64_t)cfg.split_count * d->M * d->N * sizeof(float);
    if (cfg.split_count > 65535u || need > kStaticScratchBytes) {
        set_last_error("vaicu_linear_splitk_static", "split_count * M * N * 4 bytes exceeds the 8 MiB built-in scratch");
        return VAICU_ERR_TOO_LARGE;
    }

    LinearArgs a{};
    a.I = I; a.W = W; a.bias = d->has_bias ? bias : nullptr; a.res = d->has_residual ? residual : nullptr; a.O = O;
    a.M = d->M; a.N = d->N; a.K = d->K;
    a.i_dtype = d->i_dtype; a.w_dtype = d->w_dtype; a.o_dtype = d->o_dtype; a.b_dtype = d->has_bias ? d->b_dtype : VAICU_DTYPE_NONE;
    a.has_bias = d->has_bias ? 1 : 0; a.has_res = d->has_residual ? 1 : 0;
    a.residual_order = d->residual_order; a.epilogue = d->epilogue; a.gate_fuse = 0;
    a.bias_elems = d->has_bias ? d->bias_elems : 0; a.res_elems = d->has_residual ? d->residual_elems : 0;
    a.scale = d->scalar_scale;
    // Every partial element [z, m, n] that the fold reads is written by the tile kernel
    // first, so nothing in the shared array has to start at zero.
    cudaError_t e = launch_fma_tile(a, cfg, scratch, (cudaStream_t)stream);
    if (e == cudaSuccess) e = launch_splitk_reduce(a, scratch, cfg.split_count, (cudaStream_t)stream);
    if (e != cudaSuccess) { set_last_error("vaicu_linear_splitk_static launch", cudaGetErrorString(e)); return VAICU_ERR_CUDA; }
    return VAICU_OK;
}
#pragma GCC visibility pop
