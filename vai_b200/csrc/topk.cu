// Row-wise top-k sampling over logits [M, N]: vAi's TopKSampling node
// (vai/nodes/topk-sampling.h:9-31, vai/shaders/topk-sampling.comp):
//   out[i] = sample(softmax(top-k(I[i, :]) / temperature), u)
// with the reference's exact rules: candidates ranked by (value descending, index
// ascending); Z and the running sum accumulated in that order in fp32 with the row maximum
// subtracted; the first rank whose running sum reaches u * Z is the sample (rank 0 if none).
//
// Two launches, as in the reference; the selection itself is organised for warps instead of
// workgroup-wide rounds.  Stage 1: block (g, row) owns a 2048-column slice; each of its 8 warps
// keeps 256 columns in registers (8 per lane, each lane's list sorted descending) and pops its
// own top-k in k rounds of a warp-shuffle "best head" reduction (no block barrier), leaving a
// sorted list in shared memory; warp 0 then merges the 8 sorted lists into the slice's top-k.
// Stage 2: one warp merges the G sorted candidate lists (heads in registers, lists in shared
// memory) and lane 0 samples.  Rows of at most 2048 columns need stage 1's block only.  Both
// merges are exact: the top-k of a union is within the union of the parts' top-k.  u lives in
// device memory so that a recorded launch sees each step's value.
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
    const void* logits;       // stage 1: [M, N] of dtype
    const uint2* cand_in;     // stage 2: [M, G * k] (value bits, index), G sorted lists of k
    uint2* cand_out;          // stage 1 with G > 1: [M, G * k]
    uint32_t* out;            // sampling launch: [M]
    const float* u;           // device scalar in [0, 1)
    uint32_t N;               // stage 1: row width; stage 2: lists per row (G)
    uint32_t k;               // min(K, row width of the logits)
    int32_t dtype;
    float temperature;
    // vocabulary slabs: the logits are a window of wider rows / the candidates carry global indices
    size_t ld;                // stage 1: elements between rows of the logits
    uint32_t index_base;      // stage 1: added to every column index
    // stage 2 reads list l of row r at cand_in[l * list_stride + r * row_stride] (entries)
    size_t list_stride, row_stride;
    uint32_t list_len;        // entries per list in cand_in (>= k; the tail may be padding)
    uint2* list_out;          // stage 2: write the merged, sorted k_out entries per row here instead of sampling
    uint32_t k_out;           // entries per row in list_out (>= k: the tail is padded with sentinels)
};

// One warp merges `nlists` descending lists of `len` (value, index) entries each, stored
// back to back at `lists`, into the best `k` of their union, in order, at top_v / top_i.
// Lane l walks lists l, l + 32, ...: their heads live in registers, SLOTS lists per lane at most.
template <uint32_t SLOTS>
__device__ __forceinline__ void merge_lists(const uint2* lists, uint32_t nlists, size_t stride, uint32_t len, uint32_t k, float* top_v,
                                            uint32_t* top_i, uint32_t lane)
{
    float hv[SLOTS];
    uint32_t hi[SLOTS], pos[SLOTS];
#pragma unroll
    for (uint32_t j = 0; j < SLOTS; ++j) {
        const uint32_t l = lane + 32u * j;
        pos[j] = 0u;
        if (l < nlists && len > 0u) {
            const uint2 c = lists[(size_t)l * stride];
            hv[j] = __uint_as_float(c.x); hi[j] = c.y;
        } else {
            hv[j] = kLowest; hi[j] = 0xFFFFFFFFu;
        }
    }
    for (uint32_t r = 0; r < k; ++r) {
        // this lane's best head, then the warp's
        float bv = hv[0];
        uint32_t bi = hi[0];
#pragma unroll
        for (uint32_t j = 1; j < SLOTS; ++j)
            if (outranks(hv[j], hi[j], bv, bi)) { bv = hv[j]; bi = hi[j]; }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (outranks(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0u) { top_v[r] = bv; top_i[r] = bi; }
        // the list whose head won advances (indices are unique, sentinels aside)
#pragma unroll
        for (uint32_t j = 0; j < SLOTS; ++j) {
            if (hi[j] == bi && hv[j] == bv && bi != 0xFFFFFFFFu) {
                const uint32_t l = lane + 32u * j;
                if (++pos[j] < len) {
                    const uint2 c = lists[(size_t)l * stride + pos[j]];
                    hv[j] = __uint_as_float(c.x); hi[j] = c.y;
                } else {
                    hv[j] = kLowest; hi[j] = 0xFFFFFFFFu;
                }
            }
        }
    }
    __syncwarp();
}

// Temperature softmax over the k winners and the inverse-CDF sample (topk-sampling.comp:237-258).
__device__ __forceinline__ uint32_t sample(const float* top_v, const uint32_t* top_i, uint32_t k, float temperature, float u)
{
    const float inv_t = 1.0f / fmaxf(temperature, 1e-6f);
    const float m = top_v[0];
    float z = 0.0f;
    for (uint32_t r = 0; r < k; ++r) z += expf((top_v[r] - m) * inv_t);
    const float target = u * z;
    float cum = 0.0f;
    for (uint32_t r = 0; r < k; ++r) {
        cum += expf((top_v[r] - m) * inv_t);
        if (cum >= target) return top_i[r];
    }
    return top_i[0];
}

// Stage 1.  SAMPLE: the row fits one block, which also samples.
template <bool SAMPLE>
__global__ void __launch_bounds__(kPartThreads) topk_slice_kernel(const TopkParams p)
{
    const uint32_t row = blockIdx.y, g = blockIdx.x, G = gridDim.x, tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31u;
    constexpr uint32_t kWarps = kPartThreads / 32u;
    __shared__ uint2 warp_list[kWarps * kMaxK];          // each warp's top-k, descending
    __shared__ float top_v[kMaxK];
    __shared__ uint32_t top_i[kMaxK];

    float lv[kList];
    uint32_t li[kList];
#pragma unroll
    for (uint32_t j = 0; j < kList; ++j) { lv[j] = kLowest; li[j] = 0xFFFFFFFFu; }
    const uint32_t slice = (p.N + G - 1u) / G;
    const uint32_t s0 = g * slice, s1 = (s0 + slice < p.N) ? s0 + slice : p.N;
    for (uint32_t i = s0 + tid; i < s1; i += kPartThreads) {
        const float v = load_as_f32(p.logits, p.dtype, (size_t)row * p.ld + i);
        const uint32_t gi = p.index_base + i;
        // insertion into the descending list (fully unrolled: the list stays in registers)
        if (outranks(v, gi, lv[kList - 1], li[kList - 1])) {
            lv[kList - 1] = v; li[kList - 1] = gi;
#pragma unroll
            for (int q = kList - 1; q > 0; --q) {
                if (outranks(lv[q], li[q], lv[q - 1], li[q - 1])) {
                    const float tv = lv[q]; lv[q] = lv[q - 1]; lv[q - 1] = tv;
                    const uint32_t ti = li[q]; li[q] = li[q - 1]; li[q - 1] = ti;
                }
            }
        }
    }
    // k rounds inside the warp: the best list head wins and its lane pops
    uint2* mine = warp_list + warp * p.k;
    for (uint32_t r = 0; r < p.k; ++r) {
        float bv = lv[0];
        uint32_t bi = li[0];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (outranks(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0u) mine[r] = make_uint2(__float_as_uint(bv), bi);
        if (li[0] == bi && lv[0] == bv && bi != 0xFFFFFFFFu) {
#pragma unroll
            for (uint32_t q = 0; q + 1u < kList; ++q) { lv[q] = lv[q + 1]; li[q] = li[q + 1]; }
            lv[kList - 1] = kLowest; li[kList - 1] = 0xFFFFFFFFu;
        }
    }
    __syncthreads();
    if (warp != 0u) return;
    merge_lists<1>(warp_list, kWarps, p.k, p.k, p.k, top_v, top_i, lane);
    if (SAMPLE) {
        if (lane == 0u) p.out[row] = sample(top_v, top_i, p.k, p.temperature, *p.u);
    } else if (p.list_out) {
        // the row fits this block and its sorted list is the result: k entries, then padding
        for (uint32_t r = lane; r < p.k_out; r += 32u)
            p.list_out[(size_t)row * p.k_out + r] = r < p.k ? make_uint2(__float_as_uint(top_v[r]), top_i[r])
                                                           : make_uint2(__float_as_uint(kLowest), 0xFFFFFFFFu);
    } else {
        for (uint32_t r = lane; r < p.k; r += 32u)
            p.cand_out[((size_t)row * G + g) * p.k + r] = make_uint2(__float_as_uint(top_v[r]), top_i[r]);
    }
}

// Stage 2: one warp per row merges the G sorted lists (copied to shared memory when they fit).
__global__ void __launch_bounds__(32) topk_merge_kernel(const TopkParams p, uint32_t lists_in_smem)
{
    extern __shared__ uint2 staged[];
    __shared__ float top_v[kMaxK];
    __shared__ uint32_t top_i[kMaxK];
    const uint32_t row = blockIdx.x, lane = threadIdx.x, G = p.N;
    const uint2* lists = p.cand_in + (size_t)row * p.row_stride;
    size_t stride = p.list_stride;
    if (lists_in_smem) {
        for (uint32_t i = lane; i < G * p.list_len; i += 32u) staged[i] = lists[(size_t)(i / p.list_len) * stride + i % p.list_len];
        __syncwarp();
        lists = staged;
        stride = p.list_len;
    }
    if (G <= 64u) merge_lists<2>(lists, G, stride, p.list_len, p.k, top_v, top_i, lane);
    else if (G <= 128u) merge_lists<4>(lists, G, stride, p.list_len, p.k, top_v, top_i, lane);
    else merge_lists<8>(lists, G, stride, p.list_len, p.k, top_v, top_i, lane);
    if (p.list_out) {
        for (uint32_t r = lane; r < p.k_out; r += 32u)
            p.list_out[(size_t)row * p.k_out + r] = r < p.k ? make_uint2(__float_as_uint(top_v[r]), top_i[r])
                                                           : make_uint2(__float_as_uint(kLowest), 0xFFFFFFFFu);
    } else if (lane == 0u) {
        p.out[row] = sample(top_v, top_i, p.k, p.temperature, *p.u);
    }
}

}  // namespace

// Blocks per row in stage 1 (1: single launch).
uint32_t topk_groups(uint32_t N) { return (N + kSlice - 1u) / kSlice; }

namespace {
// Stage 2 over `G` lists per row; samples into `out`, or writes the merged list to `list_out`.
cudaError_t launch_merge(const TopkParams& q, uint32_t M, uint32_t G, cudaStream_t stream)
{
    const size_t bytes = (size_t)G * q.list_len * sizeof(uint2);
    const bool in_smem = bytes <= 200u * 1024u;
    if (in_smem && bytes > 48u * 1024u) {
        static SmemOptIn optin;
        if (cudaError_t e = optin.ensure(topk_merge_kernel, (int)(200u * 1024u)); e != cudaSuccess) return e;
    }
    topk_merge_kernel<<<M, 32, in_smem ? bytes : 0, stream>>>(q, in_smem ? 1u : 0u);
    return cudaGetLastError();
}
}  // namespace

// `list_out` null: the TopKSampling node (sample into `out`).  `list_out` set: the per-slab step of a
// vocabulary-split head — the sorted top-K list of each row of this slab, indices offset by index_base.
cudaError_t launch_topk(const void* logits, int dtype, uint32_t M, uint32_t N, size_t ld, uint32_t K, uint32_t index_base,
                        float temperature, const float* u, void* workspace, uint32_t* out, void* list_out, cudaStream_t stream)
{
    TopkParams p{};
    p.logits = logits; p.dtype = dtype; p.temperature = temperature; p.u = u; p.out = out;
    p.N = N;
    p.ld = ld;
    p.index_base = index_base;
    p.k = K < N ? K : N;
    p.list_out = reinterpret_cast<uint2*>(list_out);
    p.k_out = K;
    const uint32_t G = topk_groups(N);
    if (G == 1u) {
        if (list_out) topk_slice_kernel<false><<<dim3(1, M), kPartThreads, 0, stream>>>(p);
        else topk_slice_kernel<true><<<dim3(1, M), kPartThreads, 0, stream>>>(p);
        return cudaGetLastError();
    }
    p.cand_out = reinterpret_cast<uint2*>(workspace);
    p.list_out = nullptr;                       // the slices feed stage 2
    topk_slice_kernel<false><<<dim3(G, M), kPartThreads, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    TopkParams q = p;
    q.logits = nullptr;
    q.cand_in = reinterpret_cast<const uint2*>(workspace);
    q.cand_out = nullptr;
    q.N = G;
    q.list_len = p.k;
    q.list_stride = p.k;
    q.row_stride = (size_t)G * p.k;
    q.list_out = reinterpret_cast<uint2*>(list_out);
    return launch_merge(q, M, G, stream);
}

cudaError_t launch_topk_sample(const void* logits, int dtype, uint32_t M, uint32_t N, uint32_t K, float temperature,
                               const float* u, void* workspace, uint32_t* out, cudaStream_t stream)
{
    return launch_topk(logits, dtype, M, N, N, K, 0u, temperature, u, workspace, out, nullptr, stream);
}

// Merge step of a vocabulary-split head: `groups` sorted lists per row (one per GPU, list_len entries each,
// padding allowed at the tail), list g of row m at pairs[g * group_stride + m * list_len]; keeps the best k
// of their union and samples.
cudaError_t launch_topk_merge_sample(const void* pairs, uint32_t groups, size_t group_stride, uint32_t M, uint32_t list_len,
                                     uint32_t k, float temperature, const float* u, uint32_t* out, cudaStream_t stream)
{
    TopkParams q{};
    q.cand_in = reinterpret_cast<const uint2*>(pairs);
    q.N = groups;
    q.k = k;
    q.list_len = list_len;
    q.list_stride = group_stride;
    q.row_stride = list_len;
    q.temperature = temperature;
    q.u = u;
    q.out = out;
    return launch_merge(q, M, groups, stream);
}

}  // namespace vaicu
