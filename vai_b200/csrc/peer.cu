// Kernels for a Linear whose work is split over the GPUs of one host (no counterpart in the
// single-device reference): a barrier between the ranks' streams and the fold of row-parallel
// partial sums.  Peers' memory is only ever reached with ordinary loads and stores through
// pointers opened with CUDA IPC; nothing here uses the copy engine's multicast forms.
//
//   peer_barrier_kernel   every rank runs one on its own GPU at the same point of its stream.
//                         Rank r writes the barrier's epoch into slot r of every rank's flag array
//                         and then waits until all slots of its own array carry that epoch.  What
//                         a rank stored to its peers before the barrier (in earlier kernels of the
//                         stream) is visible to them after it.  The wait is bounded: when it runs
//                         out the kernel sets the device status word and returns.
//   partial_fold_kernel   O[row0 + i, n] = scale * sum_p parts[p][i][n] (+ R[row0 + i, n]) for the rows
//                         this rank owns after a row-parallel Linear whose epilogue scattered the
//                         ranks' partial sums to their owners (vaicu_linear_run_reduce_scatter); the
//                         finished rows are stored into every rank's output, which is the all-gather.
#include "common.cuh"

namespace vaicu {

namespace {

constexpr uint32_t kBarrierSpinLimit = 1u << 19;     // each probe sleeps ~100 ns and reads over the link: about half a second

struct PeerBarrierParams {
    uint32_t* flags[8];       // flags[t]: rank t's array of `world` slots (flags[rank] is local)
    uint32_t* epoch;          // local counter of barriers passed
    int* status;
    int world, rank;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerBarrierParams p)
{
    __shared__ uint32_t s_epoch;
    if (threadIdx.x == 0) {
        s_epoch = *p.epoch + 1u;
        *p.epoch = s_epoch;
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    const int t = (int)threadIdx.x;
    if (t < p.world) {
        __threadfence_system();       // this GPU's earlier stores to peers are ordered ahead of the signal
        uint32_t* theirs = p.flags[t] + p.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
        const uint32_t* mine = p.flags[p.rank] + t;
        bool ok = false;
        for (uint32_t spin = 0; spin < kBarrierSpinLimit; ++spin) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int32_t)(seen - e) >= 0) { ok = true; break; }      // a rank may already be one barrier ahead
            __nanosleep(100);
        }
        if (!ok) atomicExch(p.status, 1);
    }
}

struct FoldParams {
    const void* parts;        // [n_parts][rows][N]
    const void* residual;     // [M, N] in o_dtype (rows row0.. are read), or null
    void* dst[8];             // [M, N] outputs; rows [row0, row0 + rows) are written in each
    uint32_t n_parts, rows, N, row0, n_dst;
    int part_dtype, o_dtype;
    float scale;
};

// Eight consecutive outputs per thread: 16- or 32-byte loads of every slab, one 16-byte (16-bit
// outputs) or two 16-byte (fp32) stores per destination, so that the rows that go to peers cross
// NVLink as whole vectors.  Needs N % 8 == 0 and 16-byte aligned bases; the scalar form below
// takes everything else.
__global__ void __launch_bounds__(256) partial_fold_vec_kernel(const FoldParams p)
{
    const size_t total = (size_t)p.rows * p.N;
    for (size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8u; e < total; e += (size_t)gridDim.x * blockDim.x * 8u) {
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t q = 0; q < p.n_parts; ++q) {
            const size_t at = (size_t)q * total + e;
            if (p.part_dtype == VAICU_DTYPE_F32) {
                const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.parts) + at);
                const float4 t0 = s[0], t1 = s[1];
                acc[0] += t0.x; acc[1] += t0.y; acc[2] += t0.z; acc[3] += t0.w;
                acc[4] += t1.x; acc[5] += t1.y; acc[6] += t1.z; acc[7] += t1.w;
            } else {
                const uint4 t = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.parts) + at);
                const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (p.part_dtype == VAICU_DTYPE_F16) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                        acc[2 * k] += f.x; acc[2 * k + 1] += f.y;
                    } else {
                        acc[2 * k] += __uint_as_float(w[k] << 16); acc[2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
                    }
                }
            }
        }
        const size_t out = (size_t)p.row0 * p.N + e;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float v = p.scale * acc[c];
            if (p.residual) v += load_as_f32(p.residual, p.o_dtype, out + c);
            acc[c] = v;
        }
        if (p.o_dtype == VAICU_DTYPE_F32) {
            const float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]), hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
            for (uint32_t d = 0; d < p.n_dst; ++d) {
                float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.dst[d]) + out);
                o[0] = lo; o[1] = hi;
            }
        } else {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (p.o_dtype == VAICU_DTYPE_F16) {
                    __half2 h = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
                    w[k] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                    __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
                    w[k] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            const uint4 packed = make_uint4(w[0], w[1], w[2], w[3]);
            for (uint32_t d = 0; d < p.n_dst; ++d) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dst[d]) + out) = packed;
        }
    }
}

__global__ void __launch_bounds__(256) partial_fold_kernel(const FoldParams p)
{
    const size_t total = (size_t)p.rows * p.N;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (uint32_t q = 0; q < p.n_parts; ++q) acc += load_as_f32(p.parts, p.part_dtype, (size_t)q * total + e);
        const size_t out = (size_t)p.row0 * p.N + e;
        float v = p.scale * acc;
        if (p.residual) v += load_as_f32(p.residual, p.o_dtype, out);
        for (uint32_t d = 0; d < p.n_dst; ++d) store_from_f32(p.dst[d], p.o_dtype, out, v);
    }
}

}  // namespace

cudaError_t launch_peer_barrier(uint32_t* const* flags, int world, int rank, uint32_t* epoch, int* status, cudaStream_t stream)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return cudaErrorInvalidValue;
    PeerBarrierParams p{};
    for (int i = 0; i < world; ++i) p.flags[i] = flags[i];
    p.epoch = epoch;
    p.status = status;
    p.world = world;
    p.rank = rank;
    peer_barrier_kernel<<<1, 32, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_partial_fold(const void* parts, uint32_t n_parts, uint32_t rows, uint32_t N, int part_dtype, const void* residual,
                                float scale, int o_dtype, void* const* dsts, uint32_t n_dst, uint32_t row0, int sm_count, cudaStream_t stream)
{
    if (n_dst < 1 || n_dst > 8) return cudaErrorInvalidValue;
    FoldParams p{};
    p.parts = parts; p.residual = residual;
    for (uint32_t i = 0; i < n_dst; ++i) p.dst[i] = dsts[i];
    p.n_parts = n_parts; p.rows = rows; p.N = N; p.row0 = row0; p.n_dst = n_dst;
    p.part_dtype = part_dtype; p.o_dtype = o_dtype; p.scale = scale;
    bool vec = (N % 8u == 0u) && ((reinterpret_cast<uintptr_t>(parts) & 15u) == 0) &&
               (!residual || (reinterpret_cast<uintptr_t>(residual) & 15u) == 0);
    for (uint32_t i = 0; i < n_dst; ++i) vec = vec && ((reinterpret_cast<uintptr_t>(dsts[i]) & 15u) == 0);
    const size_t work = vec ? ((size_t)rows * N) / 8u : (size_t)rows * N;
    size_t blocks = (work + 255u) / 256u;
    const size_t cap = (size_t)(sm_count > 0 ? sm_count : 148) * 8u;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    if (vec) partial_fold_vec_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
    else partial_fold_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace vaicu
