// Shared device/host helpers for the Linear kernels: dtype codes, element
// load/store, the epilogue functions, the bias/residual broadcast rule.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/vaicu.h"

namespace vaicu {

// Internal, fully resolved description of one Linear call; filled by the plan.
struct LinearArgs {
    const void* I;
    const void* W;
    const void* bias;
    const void* res;
    void* O;
    uint32_t M, N, K;      // N counts weight rows (2H when gate_fuse)
    int32_t i_dtype, w_dtype, o_dtype, b_dtype;
    int32_t has_bias, has_res, residual_order, epilogue, gate_fuse;
    uint32_t bias_elems, res_elems;   // 0: covers O, else index modulo (vAi linear.h:2333-2338)
    float scale;
};

__host__ __device__ inline uint32_t dtype_size(int dt) { return dt == VAICU_DTYPE_F32 ? 4u : 2u; }

__device__ __forceinline__ float load_as_f32(const void* p, int dt, size_t i)
{
    if (dt == VAICU_DTYPE_F32) return reinterpret_cast<const float*>(p)[i];
    if (dt == VAICU_DTYPE_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_f32(void* p, int dt, size_t i, float v)
{
    if (dt == VAICU_DTYPE_F32) reinterpret_cast<float*>(p)[i] = v;
    else if (dt == VAICU_DTYPE_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Epilogue functions in fp32 with the reference's constants
// (vAi vai/shaders/common/activation.h:19-58).
__device__ __forceinline__ float erf_as(float x)   // Abramowitz-Stegun 7.1.26
{
    const float t = 1.0f / (1.0f + 0.3275911f * fabsf(x));
    const float p = ((((1.061405429f * t - 1.453152027f) * t + 1.421413741f) * t - 0.284496736f) * t + 0.254829592f) * t;
    const float s = (x > 0.0f) ? 1.0f : ((x < 0.0f) ? -1.0f : 0.0f);
    return s * (1.0f - p * expf(-x * x));
}

__device__ __forceinline__ float apply_epilogue(int code, float x)
{
    switch (code) {
    case VAICU_EPILOGUE_RELU: return fmaxf(x, 0.0f);
    case VAICU_EPILOGUE_GELU: return 0.5f * x * (1.0f + erf_as(x * 0.707106781186547524400844f));
    case VAICU_EPILOGUE_GELU_TANH: {
        const float c = 0.797884560802865355879892f;
        return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
    }
    case VAICU_EPILOGUE_SILU: return x / (1.0f + expf(-x));
    case VAICU_EPILOGUE_SIGMOID: return 1.0f / (1.0f + expf(-x));
    default: return x;
    }
}

// Everything after the dot product for one output element.
struct EpilogueArgs {
    const void* bias;
    const void* res;
    int32_t b_dtype, o_dtype;
    int32_t has_bias, has_res, residual_order, epilogue;
    uint32_t bias_elems, res_elems;
    float scale;
};

__host__ __device__ inline EpilogueArgs make_epilogue_args(const LinearArgs& a)
{
    EpilogueArgs e;
    e.bias = a.bias; e.res = a.res; e.b_dtype = a.b_dtype; e.o_dtype = a.o_dtype;
    e.has_bias = a.has_bias; e.has_res = a.has_res; e.residual_order = a.residual_order;
    e.epilogue = a.epilogue; e.bias_elems = a.bias_elems; e.res_elems = a.res_elems; e.scale = a.scale;
    return e;
}

__device__ __forceinline__ float read_bias(const EpilogueArgs& e, size_t flat)
{
    if (!e.has_bias) return 0.0f;
    return load_as_f32(e.bias, e.b_dtype, e.bias_elems ? flat % e.bias_elems : flat);
}
__device__ __forceinline__ float read_res(const EpilogueArgs& e, size_t flat)
{
    if (!e.has_res) return 0.0f;
    return load_as_f32(e.res, e.o_dtype, e.res_elems ? flat % e.res_elems : flat);
}

// O = s*ep(acc + b) + R   or   s*ep(acc + b + R)   (vAi linear-slab.comp:236-241,
// linear-reduce.comp:108-112).  `flat` is the row-major index into O [M, N].
__device__ __forceinline__ float finish_output(const EpilogueArgs& e, float acc, size_t flat)
{
    const float a = acc + read_bias(e, flat);
    const float r = read_res(e, flat);
    return e.residual_order == VAICU_RESIDUAL_BEFORE_EPILOGUE ? e.scale * apply_epilogue(e.epilogue, a + r)
                                                              : e.scale * apply_epilogue(e.epilogue, a) + r;
}

// The same with the bias and residual values already in registers (read ahead of the dot product).
__device__ __forceinline__ float finish_output_pre(const EpilogueArgs& e, float acc, float bias, float res)
{
    const float a = acc + bias;
    return e.residual_order == VAICU_RESIDUAL_BEFORE_EPILOGUE ? e.scale * apply_epilogue(e.epilogue, a + res)
                                                              : e.scale * apply_epilogue(e.epilogue, a) + res;
}

// Fused Linear + GatedMul (vAi vai/nodes/gated-mul.h:9-20): gate and value
// accumulators of output column j; bias holds 2H entries, gate half first.
// `flat` indexes O [M, H]; bias index is the weight row.
__device__ __forceinline__ float finish_gated(const EpilogueArgs& e, float acc_gate, float acc_up,
                                              uint32_t j, uint32_t H, size_t flat)
{
    float g = acc_gate, u = acc_up;
    if (e.has_bias) {
        g += load_as_f32(e.bias, e.b_dtype, j);
        u += load_as_f32(e.bias, e.b_dtype, (size_t)H + j);
    }
    return e.scale * (apply_epilogue(e.epilogue, g) * u) + read_res(e, flat);
}

// Argmax bookkeeping shared by the Argmax kernels and the weight-streaming kernel's fused form:
// the larger value wins, the LOWER index among equal values (what torch.argmax, the reference's
// test oracle, returns); a NaN never wins.  kArgmaxLowest is the shader's start value
// (vAi vai/shaders/argmax.comp:58).
constexpr float kArgmaxLowest = -3.4028235e38f;
__device__ __forceinline__ void argmax_take(float v, uint32_t i, float& best, uint32_t& idx)
{
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
}
// v as it reads back after being stored in dtype dt.
__device__ __forceinline__ float round_through(int dt, float v)
{
    if (dt == VAICU_DTYPE_F16) return __half2float(__float2half_rn(v));
    if (dt == VAICU_DTYPE_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}

// The Argmax node folded into the weight-streaming Linear that feeds it: every block keeps the
// best (value, column) of the outputs it produces, the last block to finish folds the blocks'
// candidates.  `count` must be zero when the kernel starts and is zero again when it ends.
struct GemvArgmax {
    float* block_val;          // [grid][M]
    uint32_t* block_idx;       // [grid][M]
    unsigned int* count;       // blocks done
    float* out_val;            // [M] or null
    uint32_t* out_idx;         // [M]
    uint32_t index_base;       // added to every column index (first vocabulary entry of a slab)
    int write_logits;          // also store O
};

// Launchers implemented in the .cu files; each returns a cudaError_t.
struct GemvConfig { int rows_per_warp; int k_warps; int grid; size_t smem; int vectorized; int unroll; int plain_launch; };

cudaError_t launch_gemv(const LinearArgs& a, const GemvConfig& cfg, cudaStream_t stream, const GemvArgmax* argmax = nullptr);
// `tuning` (may be null) carries a caller's overrides of the geometry; see vaicu_linear_tuning.
GemvConfig  choose_gemv(const LinearArgs& a, int sm_count, bool w_aligned16, const vaicu_linear_tuning* tuning = nullptr);
// `a` describes the concatenation (a.N = sum of rows); plain Linears only.
cudaError_t launch_gemv_group(const LinearArgs& a, const GemvConfig& cfg, uint32_t nseg, const uint32_t* rows,
                              const void* const* w, void* const* o, cudaStream_t stream);

struct FmaTileConfig { uint32_t split_count, split_size; };
cudaError_t launch_fma_tile(const LinearArgs& a, const FmaTileConfig& cfg, float* partial, cudaStream_t stream);
cudaError_t launch_splitk_reduce(const LinearArgs& a, const float* partial, uint32_t split_count, cudaStream_t stream);
// partial [splits][M][sum of rows] -> the members' dense outputs (rows[i] % 4 == 0, O[i] 16-byte aligned)
cudaError_t launch_group_fold(const float* partial, uint32_t splits, uint32_t M, uint32_t count, const uint32_t* rows,
                              void* const* O, int o_dtype, cudaStream_t stream);
cudaError_t launch_cast_f32_to_16(const float* src, void* dst, int dst_dtype, size_t n, int sm_count, cudaStream_t stream);

cudaError_t launch_argmax(const void* in, int dtype, uint32_t M, uint32_t N, uint32_t* out, cudaStream_t stream);
uint32_t argmax_parts(uint32_t N);
uint32_t topk_groups(uint32_t N);
cudaError_t launch_topk_sample(const void* logits, int dtype, uint32_t M, uint32_t N, uint32_t K, float temperature,
                               const float* u, void* workspace, uint32_t* out, cudaStream_t stream);
cudaError_t launch_topk(const void* logits, int dtype, uint32_t M, uint32_t N, size_t ld, uint32_t K, uint32_t index_base,
                        float temperature, const float* u, void* workspace, uint32_t* out, void* list_out, cudaStream_t stream);
cudaError_t launch_topk_merge_sample(const void* pairs, uint32_t groups, size_t group_stride, uint32_t M, uint32_t list_len,
                                     uint32_t k, float temperature, const float* u, uint32_t* out, cudaStream_t stream);
cudaError_t launch_argmax_pairs(const void* in, int dtype, uint32_t M, uint32_t N, size_t ld, uint32_t index_base, void* workspace,
                                float* out_val, uint32_t* out_idx, cudaStream_t stream);
cudaError_t launch_argmax_merge(const float* vals, const uint32_t* idxs, uint32_t groups, size_t group_stride, uint32_t M,
                                float* out_val, uint32_t* out_idx, cudaStream_t stream);

cudaError_t launch_rms_norm(const void* in, const void* scale, const void* shift, const void* res, void* out, uint32_t rows,
                            uint32_t feat, int i_dtype, int w_dtype, int o_dtype, float eps, int sm_count, cudaStream_t stream);
cudaError_t launch_layer_norm(const void* in, const void* scale, const void* shift, const void* res, void* out, uint32_t rows,
                            uint32_t feat, int i_dtype, int w_dtype, int o_dtype, float eps, int sm_count, cudaStream_t stream);

cudaError_t launch_peer_barrier(uint32_t* const* flags, int world, int rank, uint32_t* epoch, int* status, cudaStream_t stream);
cudaError_t launch_partial_fold(const void* parts, uint32_t n_parts, uint32_t rows, uint32_t N, int part_dtype, const void* residual,
                                float scale, int o_dtype, void* const* dsts, uint32_t n_dst, uint32_t row0, int sm_count, cudaStream_t stream);
cudaError_t launch_gated_mul(const void* in, void* out, uint32_t rows, uint32_t H, int i_dtype, int o_dtype, int act,
                             int sm_count, cudaStream_t stream);

// Programmatic dependent launch: the kernel after this one in the stream may start its prologue
// as soon as every block here has passed launch_dependents(); a kernel launched that way must not
// touch what its predecessor writes (or write what it reads) before dependency_wait() returns
// (predecessor complete, its writes visible).  Both are no-ops for a plain launch.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with programmatic stream serialization allowed (only for kernels that call
// dependency_wait() before their first dependent access).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args)
{
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, kern, std::forward<Args>(args)...);
}

// The same, as thread-block clusters of `cluster` CTAs along x (the grid is a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster,
                               Args&&... args)
{
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    lc.attrs = attr;
    lc.numAttrs = 2;
    return cudaLaunchKernelEx(&lc, kern, std::forward<Args>(args)...);
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device property of a kernel: a process
// that drives several GPUs has to opt in on each of them.  One flag per device ordinal and
// kernel instantiation; the attribute call itself is idempotent, so a race between two threads
// on the first launch only repeats it.
struct SmemOptIn {
    static constexpr int kMaxDevices = 64;
    unsigned char done[kMaxDevices] = {};
    template <typename Kernel> cudaError_t ensure(Kernel kern, int bytes)
    {
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const bool tracked = dev >= 0 && dev < kMaxDevices;
        if (tracked && done[dev]) return cudaSuccess;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess && tracked) done[dev] = 1;
        return e;
    }
};

// Records "<where>: <what>" as the calling thread's last error text
// (vaicu_last_cuda_error).
void set_last_error(const char* where, const char* what);

}  // namespace vaicu
