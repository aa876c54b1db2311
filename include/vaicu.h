/* vaicu.h — C ABI of the B200 (sm_100a) backend for vAi's Linear node.
 *
 * This is the whole surface a host binds to replace the Vulkan device layer
 * on the `vai::node::Linear` path.  Every function returns an int status
 * (VAICU_OK == 0); nothing aborts or throws across this boundary.  All data
 * pointers handed to vaicu_linear_run() are DEVICE pointers owned by the
 * caller; the library never frees or keeps them.  There is no CPU fallback:
 * a call that cannot run on the GPU returns an error status.
 *
 * Each declaration names the reference interface it stands in for
 * (path inside the vAi source tree : line).
 */
#ifndef VAICU_H
#define VAICU_H

#include <stddef.h>
#include <stdint.h>

/* Only the functions below are exported from libvaicu.so. */
#if defined(__GNUC__)
#define VAICU_API __attribute__((visibility("default")))
#else
#define VAICU_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
    VAICU_OK                 = 0,
    VAICU_ERR_INVALID_VALUE  = 1,  /* null pointer, bad enum, bad shape        */
    VAICU_ERR_UNSUPPORTED    = 2,  /* dtype combination with no kernel         */
    VAICU_ERR_CUDA           = 3,  /* a CUDA runtime/driver call failed        */
    VAICU_ERR_NO_DEVICE      = 4,  /* no sm_100 device / driver present        */
    VAICU_ERR_WORKSPACE      = 5,  /* workspace null or too small              */
    VAICU_ERR_ALIGNMENT      = 6,  /* pointer not aligned to its element size  */
    VAICU_ERR_TOO_LARGE      = 7,  /* shape beyond a fixed-capacity entry point */
    VAICU_ERR_TIMEOUT        = 8   /* a bounded device-side wait gave up       */
};

/* vai::Dtype crosses the host/kernel boundary as an integer
 * (vai/engine/tensor.h:19, vai/shaders/common/spec_constants.h:6-8).
 * Fp32, Fp16 and None keep their reference values; bf16 is appended. */
enum {
    VAICU_DTYPE_F32  = 0,
    VAICU_DTYPE_F16  = 1,
    VAICU_DTYPE_NONE = 2,
    VAICU_DTYPE_BF16 = 3
};

/* vai::Epilogue (vai/nodes/common.h:31-39; codes of
 * vai/shaders/common/activation.h:8). */
enum {
    VAICU_EPILOGUE_NONE      = 0,
    VAICU_EPILOGUE_RELU      = 1,
    VAICU_EPILOGUE_GELU      = 2,
    VAICU_EPILOGUE_GELU_TANH = 3,
    VAICU_EPILOGUE_SILU      = 4,
    VAICU_EPILOGUE_SIGMOID   = 5
};

/* vai::ResidualOrder (vai/nodes/common.h:42-45). */
enum {
    VAICU_RESIDUAL_AFTER_EPILOGUE  = 0,
    VAICU_RESIDUAL_BEFORE_EPILOGUE = 1
};

/* Kernel families a plan can resolve to (reported by vaicu_linear_plan_info;
 * the analogue of the pipeline name chosen in Linear::prepare(),
 * vai/nodes/linear.h:2355-2666). */
enum {
    VAICU_KERNEL_GEMV     = 1,  /* M <= 8 weight-streaming kernel ("slab")     */
    VAICU_KERNEL_FMA_TILE = 2,  /* fp32 FFMA tile GEMM (exact fp32, any shape) */
    VAICU_KERNEL_TC_GEMM  = 3,  /* tcgen05/TMEM GEMM, activations on UMMA-M    */
    VAICU_KERNEL_TC_SKINNY= 4   /* tcgen05/TMEM GEMM, weights on UMMA-M (swap) */
};

typedef struct vaicu_device      vaicu_device;
typedef struct vaicu_buffer      vaicu_buffer;
typedef struct vaicu_linear_plan vaicu_linear_plan;
/* A stream handle is a cudaStream_t passed as void* (NULL = default stream). */
typedef void* vaicu_stream_t;

/* Everything Linear::prepare() freezes for one recording
 * (vai/nodes/linear.h:2291-2353 and the spec/push constants of
 * linear.h:2371-2386, 2677-2685, 2726, 2793).
 *
 *   O = s * epilogue(I . W^T + bias) + R        residual_order AFTER
 *   O = s * epilogue(I . W^T + bias + R)        residual_order BEFORE
 *
 * I [M,K], W [N,K], O [M,N] dense row-major.  With gate_fuse != 0 the weight
 * holds 2H rows (gate rows [0,H), value rows [H,2H), N == 2H) and the output
 * is [M,H]: O = s * (epilogue(acc_gate + bias_gate) * (acc_up + bias_up)),
 * the Linear followed by vai's GatedMul (vai/nodes/gated-mul.h:9-20) in one
 * pass (no residual; a bias, if any, has one entry per weight row).  bias_elems / residual_elems: 0 means "covers O"; otherwise the
 * operand has that many elements and is read at (flat index % elems)
 * (linear.h:2333-2338). */
typedef struct vaicu_linear_desc {
    uint32_t M, N, K;
    int32_t  i_dtype, w_dtype, o_dtype, b_dtype;
    int32_t  has_bias;
    uint32_t bias_elems;
    int32_t  has_residual;
    uint32_t residual_elems;
    int32_t  residual_order;
    int32_t  epilogue;
    float    scalar_scale;
    uint32_t split_size;     /* 0: library heuristic; else K span per split, >= 32 */
    int32_t  gate_fuse;
} vaicu_linear_desc;

typedef struct vaicu_linear_info {
    int32_t  kernel;         /* VAICU_KERNEL_*                                  */
    uint32_t split_count;    /* K splits (1 = none)                             */
    uint32_t tile_m, tile_n; /* CTA tile (rows of O, columns of O); 0 for GEMV  */
    uint32_t launches;       /* kernels one vaicu_linear_run() enqueues         */
    size_t   workspace_bytes;
} vaicu_linear_info;

/* ---- device (replaces eva::Device; vai/engine/neural-net.h:251-257) ------ */
VAICU_API int  vaicu_device_open(int ordinal, vaicu_device** out);
VAICU_API int  vaicu_device_close(vaicu_device* dev);
VAICU_API int  vaicu_device_sm_count(const vaicu_device* dev, int* out);   /* eva::Device::computeBlockCount(), linear.h:613 */
VAICU_API int  vaicu_device_synchronize(vaicu_device* dev);
/* Synchronises the device and reads (then clears) the word the kernels set when
 * one of their bounded waits ran out: *out != 0 and VAICU_ERR_TIMEOUT in that
 * case.  Stands in for the lost-device report of NeuralNet::sync()
 * (vai/engine/neural-net.cpp:206-217). */
VAICU_API int  vaicu_device_status(vaicu_device* dev, int* out);

/* Self-test of that report: enqueues one single-warp kernel that waits, with a limit of 1024
 * probes, on a barrier nothing ever arrives on, gives up, and sets the status word exactly as
 * the GEMM kernels do when one of their waits runs out; it holds no memory in flight and
 * returns normally, so the context stays usable.  The next vaicu_device_status() reports
 * VAICU_ERR_TIMEOUT once and clears the word.  For hosts that want to verify their handling of
 * a lost step (the reference's counterpart is the device-lost branch of NeuralNet::sync(),
 * vai/engine/neural-net.cpp:206-217) without anything actually going wrong. */
VAICU_API int  vaicu_device_selftest_wait_expiry(vaicu_device* dev, vaicu_stream_t stream);

/* ---- buffers (replace eva::Buffer / BufferPool::requestBuffer,
 *      vai/engine/buffer-pool.h:77-134) ---------------------------------- */
VAICU_API int   vaicu_buffer_alloc(vaicu_device* dev, size_t bytes, vaicu_buffer** out);
VAICU_API int   vaicu_buffer_free(vaicu_buffer* buf);
VAICU_API void* vaicu_buffer_ptr(const vaicu_buffer* buf);
VAICU_API size_t vaicu_buffer_size(const vaicu_buffer* buf);

/* Host<->device copies (replace the staging copy of
 * NeuralNet::prepareInputs, vai/engine/neural-net.cpp:219-280, and
 * Tensor::downloadToHost, vai/engine/tensor.cpp:459-489). Asynchronous on
 * `stream` when the host memory is pinned. */
VAICU_API int vaicu_memcpy_h2d(void* dst_device, const void* src_host, size_t bytes, vaicu_stream_t stream);
VAICU_API int vaicu_memcpy_d2h(void* dst_host, const void* src_device, size_t bytes, vaicu_stream_t stream);
VAICU_API int vaicu_memset(void* dst_device, int value, size_t bytes, vaicu_stream_t stream);
VAICU_API int vaicu_host_alloc_pinned(size_t bytes, void** out);
VAICU_API int vaicu_host_free_pinned(void* p);

/* ---- streams (replace eva::CommandBuffer submit + TimelineSemaphore,
 *      vai/engine/neural-net.h:432-438, neural-net.cpp:206-217) ----------- */
VAICU_API int vaicu_stream_create(vaicu_device* dev, vaicu_stream_t* out);
VAICU_API int vaicu_stream_sync(vaicu_stream_t stream);
VAICU_API int vaicu_stream_destroy(vaicu_stream_t stream);
/* Orders `waiter` after everything enqueued so far on `signaler` (an event record +
 * wait; also valid while `signaler` is being captured, which pulls `waiter` into the
 * recording).  Stands in for the buffer barriers between independent dispatches of one
 * command buffer (linear.h:2746): nodes that do not depend on each other may run on
 * side streams and join again. */
VAICU_API int vaicu_stream_wait_stream(vaicu_stream_t waiter, vaicu_stream_t signaler);

/* ---- events (replace the timestamp queries of NodeProfiler,
 *      vai/engine/node-profiler.h:118-178) --------------------------------- */
typedef struct vaicu_event vaicu_event;
VAICU_API int vaicu_event_create(vaicu_event** out);
VAICU_API int vaicu_event_record(vaicu_event* ev, vaicu_stream_t stream);
VAICU_API int vaicu_event_synchronize(vaicu_event* ev);
/* Milliseconds between two recorded, completed events. */
VAICU_API int vaicu_event_elapsed_ms(vaicu_event* start, vaicu_event* stop, float* out_ms);
VAICU_API int vaicu_event_destroy(vaicu_event* ev);

/* ---- recorded launches (replace the command buffer that is recorded once and
 *      resubmitted while shapes repeat, vai/engine/neural-net.h:391-438) --- */
typedef struct vaicu_graph vaicu_graph;
/* Everything enqueued on `stream` between begin and end is captured instead of
 * executed; end returns an executable recording. */
VAICU_API int vaicu_graph_capture_begin(vaicu_stream_t stream);
VAICU_API int vaicu_graph_capture_end(vaicu_stream_t stream, vaicu_graph** out);
VAICU_API int vaicu_graph_launch(vaicu_graph* graph, vaicu_stream_t stream);
VAICU_API int vaicu_graph_destroy(vaicu_graph* graph);

/* ---- the Linear plan (replaces Linear::prepare(), linear.h:2291-2704,
 *      and the PipelinePool lookup, vai/engine/pipeline-pool.h:86-116) ---- */
VAICU_API int vaicu_linear_plan_create(vaicu_device* dev, const vaicu_linear_desc* desc, vaicu_linear_plan** out);
/* Same, but with the kernel family fixed by the caller (VAICU_KERNEL_*) instead
 * of chosen by shape; VAICU_ERR_UNSUPPORTED when that family cannot run the
 * desc.  The counterpart of the reference's per-node overrides such as
 * Linear::setAccDtype (linear.h:291); used by the parity tests to drive every
 * kernel over the same shapes. */
VAICU_API int vaicu_linear_plan_create_forced(vaicu_device* dev, const vaicu_linear_desc* desc, int kernel, vaicu_linear_plan** out);
/* Same again with every choice the library would make from the shape open to the caller: a
 * field left at 0 (tc_pair / tc_wide: at -1) keeps the library's choice.  This is how the
 * parity tests reach each tile form on small shapes and how a host pins a geometry it has
 * measured; nothing is read from the environment.  The reference's counterpart is the set of
 * per-node overrides and vendor tables in Linear::prepare (linear.h:2395-2666).
 * VAICU_ERR_INVALID_VALUE for a value outside the ranges given here. */
typedef struct vaicu_linear_tuning {
    int32_t  kernel;        /* VAICU_KERNEL_*; 0: by shape                                      */
    int32_t  tc_pair;       /* 1: CTA pairs (cta_group::2, 256-row tiles); 0: single CTAs; -1   */
    int32_t  tc_wide;       /* 1: single CTA with two 128-row accumulators; 0: off; -1          */
    uint32_t tc_bn;         /* UMMA N of the unswapped kernel: multiple of 16 in 16..256; 0     */
    uint32_t tc_splits;     /* number of K splits of the tensor-core kernels; 0                 */
    int32_t  gemv_rows;     /* weight rows per warp step: 2 or 4; 0                             */
    int32_t  gemv_k_warps;  /* warps of a block that split K: 1, 2, 4 or 8; 0                   */
    int32_t  gemv_unroll;   /* k-steps in flight per lane at M = 1: 2 or 4; 0                   */
    int32_t  gemv_grid;     /* blocks of the weight-streaming kernel; 0                         */
    int32_t  gemv_plain_launch; /* 1: no programmatic dependent launch (plain stream order)     */
    int32_t  tc_fold;           /* split-K of the single-CTA tensor-core kernels: 1 = the CTAs that hold a
                                   tile's splits fold it together inside the kernel through global memory
                                   (one launch; measured slower on B200 than the dependent fold launch),
                                   2 = a second launch folds, 3 = the splits of a tile run as one cluster
                                   of 2, 4 or 8 CTAs (tc_splits, if given) and fold through distributed
                                   shared memory (swapped kernel; measured no faster than 2); 0: 2   */
    int32_t  tc_tail_strips;    /* CTA-pair kernel: column strips per tile in the last, partial round of
                                   tiles: 1 = none, 2 or 4; 0: the widest that fits the idle clusters     */
    uint32_t tc_tile_rows;      /* swapped tensor-core kernel: weight rows per tile, a multiple of 8 up to
                                   128 (the MMA stays 128 rows tall; shorter tiles spread a layer with few
                                   weight rows over all SMs); 0                                   */
    uint32_t tc_stages;         /* tensor-core kernels: at most this many stages in the shared-memory ring
                                   (2..8); 0: as many as fit                                       */
} vaicu_linear_tuning;
VAICU_API int vaicu_linear_plan_create_tuned(vaicu_device* dev, const vaicu_linear_desc* desc, const vaicu_linear_tuning* tuning,
                                             vaicu_linear_plan** out);
VAICU_API int vaicu_linear_plan_destroy(vaicu_linear_plan* plan);
VAICU_API int vaicu_linear_plan_info(const vaicu_linear_plan* plan, vaicu_linear_info* out);
/* What the most recent vaicu_linear_run on this plan enqueued: *kernel = VAICU_KERNEL_* (0 before
 * the first run), *vectorized = 1 for the 16-byte-vector / TMA form of that kernel.  A tensor may be
 * a view at an element offset into a larger buffer (vai/engine/tensor.h:228-242); operands that
 * are not 16-byte aligned make a run take the element-wise weight-streaming kernel or the FMA
 * tile kernel instead of the one the plan names, with the same results.  The reference has no
 * such query: its shaders index by element and never need the distinction. */
VAICU_API int vaicu_linear_plan_last_run(const vaicu_linear_plan* plan, int* kernel, int* vectorized);
/* Size of the "partial" temporary slot (linear.h:2697-2698) plus any private
 * staging the chosen kernel needs; 0 when the kernel needs none. */
VAICU_API int vaicu_linear_workspace_bytes(const vaicu_linear_plan* plan, size_t* out);

/* Replaces Linear::run() (linear.h:2706-2798): enqueues the plan's kernels on
 * `stream`; no allocation, no synchronisation.  `bias` / `residual` may be
 * NULL when the desc says they are absent; `workspace` may be NULL when
 * vaicu_linear_workspace_bytes() reported 0. */
VAICU_API int vaicu_linear_run(vaicu_linear_plan* plan, vaicu_stream_t stream,
                     const void* I, const void* W, const void* bias, const void* residual,
                     void* O, void* workspace);

/* A Linear and the Argmax node that reads its output (the lm_head and the greedy-decode node,
 * vai/nodes/argmax.h:9-18) as ONE launch of the weight-streaming kernel: every block keeps the best
 * (value, column) of the outputs it produces and the last block to finish folds the blocks'
 * candidates, so the logits are never read back.  Same result as vaicu_linear_run followed by
 * vaicu_argmax_run over O: values compared as stored in o_dtype, lowest index among equal maxima.
 *   O                 the logits [M, N], or NULL to skip storing them
 *   argmax_workspace  vaicu_linear_argmax_workspace_bytes(plan) bytes, 256-byte aligned; its first
 *                     256 bytes must be zero before the FIRST call (vaicu_memset) and are zero again
 *                     after every call, so a recorded launch replays without a clear
 *   index_base        added to every column index: the first vocabulary entry of this GPU's slab
 *   out_val           [M] fp32 maxima, or NULL; out_u32 [M] indices.  A column-split head passes both and
 *                     folds the ranks' candidates with vaicu_argmax_merge_run.
 * workspace_bytes reports 0 and run returns VAICU_ERR_UNSUPPORTED for plans that are not on the
 * weight-streaming kernel (M > 8, or M = 5..8 with 16-bit weights), for gated plans, and for I / W
 * views that are not 16-byte aligned; the caller then records the two nodes separately.  Two calls that
 * share a workspace must not overlap on the GPU.  No counterpart in the reference, which records one
 * dispatch per node. */
VAICU_API int vaicu_linear_argmax_workspace_bytes(const vaicu_linear_plan* plan, size_t* out_bytes);
VAICU_API int vaicu_linear_run_argmax(vaicu_linear_plan* plan, vaicu_stream_t stream, const void* I, const void* W,
                                      const void* bias, const void* residual, void* O, void* argmax_workspace,
                                      uint32_t index_base, float* out_val, void* out_u32);

/* Two or three Linears that read the same activations (q / k / v of a block) as ONE
 * Linear over their weight rows side by side: plans[i] was created for W[i] -> O[i]; all
 * must be plain (no bias, epilogue, residual, scale or gate), share M, K and dtypes, and
 * resolve to the same kernel, with 16-byte aligned operands:
 *   - the weight-streaming kernel: one launch, no workspace;
 *   - the swapped tensor-core kernel (8 < M <= 128), every N a multiple of 128: one GEMM
 *     launch that leaves fp32 partial sums of all members plus one fold that stores the
 *     members' outputs (where three runs would be three GEMMs and three folds); fp32
 *     activations are rounded to the weights' type once.  Needs `workspace` of
 *     vaicu_linear_group_workspace_bytes (256-byte aligned);
 *   - the CTA-pair tensor-core kernel (M > 128), every N a multiple of 256, 16-bit activations: one
 *     GEMM over the members' 256-column tiles, each stored to its member (fewer partial rounds of
 *     tiles than three launches); no workspace.
 * Returns VAICU_ERR_UNSUPPORTED otherwise, and the caller issues the runs one by one.
 * The first plan keeps the group's state (TMA descriptors by weight pointer); it must
 * outlive the other members' use in groups.  No counterpart in the reference, which records
 * one dispatch per node (linear.h:2706-2748); this only removes launch latency and idle SMs
 * between sibling nodes. */
VAICU_API int vaicu_linear_group_workspace_bytes(vaicu_linear_plan* const* plans, int count, size_t* out_bytes);
VAICU_API int vaicu_linear_run_group(vaicu_linear_plan* const* plans, int count, vaicu_stream_t stream,
                                     const void* I, const void* const* W, void* const* O, void* workspace);

/* Column-split Linear whose output slab is written straight into wider buffers: element
 * (m, j) of the plan's output goes to dsts[i][m * ldo + col0 + j] for every i < n_dst
 * (1..8).  With dsts = {this GPU's [M, N_full] output, its peers' outputs opened through
 * vaicu_ipc_open} the epilogue of the tensor-core kernel performs the all-gather itself
 * with plain stores over NVLink, tile by tile, instead of a collective after the kernel;
 * the ranks still need one synchronisation before anyone reads the gathered output.
 * Tensor-core plans without split-K and without residual only (VAICU_ERR_UNSUPPORTED
 * otherwise); destinations 16-byte aligned.  No counterpart in the single-device reference. */
VAICU_API int vaicu_linear_run_scatter(vaicu_linear_plan* plan, vaicu_stream_t stream, const void* I, const void* W,
                                       const void* bias, void* const* dsts, int n_dst, uint32_t ldo, uint32_t col0,
                                       void* workspace);
/* A Linear whose whole (dense) output is written to n_dst buffers at once (1..8): this GPU's and, through
 * vaicu_ipc_open, its peers'.  With dsts[i] = the address of this rank's row block inside rank i's
 * [M_total, N] tensor, ranks that each run the Linear on their own rows of the activations assemble the
 * full result everywhere inside their GEMM epilogues (an all-gather along rows, as a sequence-parallel
 * block needs in front of its column-split MLP).  Bias, epilogue, residual and scale as in
 * vaicu_linear_run (they index the plan's own [M, N]).  Tensor-core plans without split-K only;
 * destinations 16-byte aligned; the ranks synchronise (vaicu_peer_barrier_run) before anyone reads.
 * No counterpart in the single-device reference. */
VAICU_API int vaicu_linear_run_broadcast(vaicu_linear_plan* plan, vaicu_stream_t stream, const void* I, const void* W,
                                         const void* bias, const void* residual, void* const* dsts, int n_dst,
                                         void* workspace);
/* Row-parallel Linear (this GPU holds a slice of K: columns [k0, k1) of W and of the activations) whose
 * partial sums go straight to the GPUs that will fold them: row m of the plan's [M, N] output belongs to
 * GPU m / (M / n_dst), and the epilogue stores it, tile by tile with plain stores over NVLink, into that
 * GPU's staging buffer at dsts[owner][(slot * M / n_dst + m % (M / n_dst)) * N + n], in the plan's o_dtype.
 * Every staging buffer holds n_dst slabs of [M / n_dst, N]; `slot` is this rank.  The reduce-scatter of a
 * tensor-parallel MLP thereby overlaps the GEMM instead of following it.  After a vaicu_peer_barrier_run
 * each GPU folds its slabs with vaicu_partial_fold_run.  Plain tensor-core plans only (no bias, epilogue,
 * residual, scale, gate or split-K: those belong to the fold); M divisible by n_dst; 16-byte aligned
 * destinations.  No counterpart in the single-device reference. */
VAICU_API int vaicu_linear_run_reduce_scatter(vaicu_linear_plan* plan, vaicu_stream_t stream, const void* I, const void* W,
                                              void* const* dsts, int n_dst, int slot, void* workspace);
/* The fold after it: O[row0 + i, n] = scale * sum over p < n_parts of parts[p][i][n] (+ residual[row0 + i, n]),
 * i < rows, parts [n_parts][rows][N] in part_dtype (summed in fp32, in slab order), residual and outputs [.., N]
 * in o_dtype; the finished rows are stored into every dsts[d] (this GPU's output and its peers': the
 * all-gather of the row slabs), followed by another vaicu_peer_barrier_run before anyone reads them. */
VAICU_API int vaicu_partial_fold_run(vaicu_device* dev, vaicu_stream_t stream, const void* parts, uint32_t n_parts, uint32_t rows,
                                     uint32_t N, int part_dtype, const void* residual, float scale, int o_dtype,
                                     void* const* dsts, int n_dst, uint32_t row0);
/* Barrier between the streams of the `world` (<= 8) GPUs of a split Linear, as one single-warp kernel per
 * GPU: rank r stores the next epoch into slot r of every rank's flag array (flag_arrays[t], `world`
 * uint32 each, zero at the start, shared through vaicu_ipc_*), then waits until every slot of its own
 * array has reached that epoch.  Stores a rank made to its peers in earlier kernels of its stream are
 * visible to them behind the barrier.  epoch_counter is 4 bytes of this GPU's memory, zero at the start.
 * All ranks must enqueue their barriers in the same order.  The wait is bounded (about half a second):
 * when a peer never arrives the kernel sets the status word read by vaicu_device_status and returns. */
VAICU_API int vaicu_peer_barrier_run(vaicu_device* dev, vaicu_stream_t stream, void* const* flag_arrays, int world, int rank,
                                     void* epoch_counter);

/* Share a vaicu_buffer_alloc'ed range with the other processes of this host: export fills a
 * 64-byte handle to send to them, open maps a peer's range into this process (peer access
 * over NVLink), close unmaps it.  No counterpart in the reference. */
VAICU_API int vaicu_ipc_export(const void* device_ptr, void* handle64);
VAICU_API int vaicu_ipc_open(const void* handle64, void** out_ptr);
VAICU_API int vaicu_ipc_close(void* ptr);

/* Split-K Linear that allocates nothing (no counterpart in the reference, whose
 * engine always has a buffer pool to draw the "partial" slot from).
 *
 * For hosts that cannot obtain device memory at call time: processes that carve
 * up the whole device heap at start-up and forbid allocation afterwards, and
 * plugin hosts that expose no allocator.  They pass the operands they already
 * own; the fp32 partial sums go to an 8 MiB array built into the library (held
 * by every GPU that loads the library until exit), so the call is limited to
 * split_count * M * N * 4 <= 8 MiB and returns VAICU_ERR_TOO_LARGE beyond that.
 * It runs the fp32 FFMA tile kernel with K split per desc->split_size (0: a
 * per-shape choice) and the fold + bias/epilogue/residual/scale pass; gate_fuse
 * is not offered.  It calls no cudaMalloc / cudaFree and no other allocator.
 *
 * The first call on each device looks the array's address up
 * (cudaGetSymbolAddress, with that device current); make that first call before
 * any stream capture.  All calls share the one array and it keeps whatever the
 * previous call left: calls that overlap on the GPU (different streams) race;
 * calls on one stream, or otherwise ordered, are safe.  Nothing needs clearing:
 * every partial the fold reads is written first by the same call. */
VAICU_API int vaicu_linear_splitk_static(const vaicu_linear_desc* desc, vaicu_stream_t stream,
                                         const void* I, const void* W, const void* bias, const void* residual,
                                         void* O);

/* RMS normalisation over the last axis: vAi's RmsNorm node, the producer of a Linear's
 * activations in the Llama / Gemma blocks (vai/nodes/rms-norm.h:9-24, 100-170;
 * vai/shaders/rms-norm.comp):
 *   O[i,j] = I[i,j] * rsqrt(mean(I[i,:]^2) + eps) (* scale[j]) (+ shift[j]) (+ R[i,j])
 * I, R in i_dtype, scale / shift [feat] in w_dtype (either may be NULL), O in o_dtype;
 * the row statistic is accumulated in fp32.  A 16-bit o_dtype feeds the tensor-core
 * Linear without its fp32 -> 16-bit staging pass.  Enqueues one kernel. */
VAICU_API int vaicu_rms_norm_run(vaicu_device* dev, vaicu_stream_t stream, const void* in, const void* scale,
                                 const void* shift, const void* residual, void* out, uint32_t rows, uint32_t feat,
                                 int i_dtype, int w_dtype, int o_dtype, float eps);

/* Layer normalisation over the last axis: vAi's LayerNorm node, the producer of a Linear's
 * activations in the GPT-2 blocks (vai/nodes/layer-norm.h:9-31, 91-160;
 * vai/shaders/layer-norm.comp):
 *   O[i, j] = (I[i, j] - mean_i) * rsqrt(var_i + eps) * scale[j] (+ shift[j]) (+ R[i, j])
 * with biased variance and fp32 statistics whatever the dtypes.  Arguments as for
 * vaicu_rms_norm_run; `scale` is required, `shift` and `residual` may be NULL. */
VAICU_API int vaicu_layer_norm_run(vaicu_device* dev, vaicu_stream_t stream, const void* in, const void* scale,
                                 const void* shift, const void* residual, void* out, uint32_t rows, uint32_t feat,
                                 int i_dtype, int w_dtype, int o_dtype, float eps);

/* vAi's GatedMul node as a launch of its own (vai/nodes/gated-mul.h:9-20, 56-84;
 * vai/shaders/gated-mul.comp:38-49):
 *   O[r, j] = activation(I[r, j]) * I[r, H + j]      I [rows, 2H] -> O [rows, H]
 * `activation` is a VAICU_EPILOGUE_* code (silu: SwiGLU, gelu: GEGLU, relu: ReGLU, none:
 * bilinear), evaluated in fp32 with the reference's constants.  A host engine records a
 * gate|value Linear followed by this node as one vaicu_linear_run with desc.gate_fuse set;
 * this entry is what it records when the pair cannot be merged.  Enqueues one kernel. */
VAICU_API int vaicu_gated_mul_run(vaicu_device* dev, vaicu_stream_t stream, const void* in, void* out, uint32_t rows,
                                  uint32_t H, int i_dtype, int o_dtype, int activation);

/* Row-wise argmax of logits [M, N] (fp32 / fp16 / bf16) into M raw uint32 indices:
 * vAi's Argmax node, the greedy-decode consumer of the lm_head Linear
 * (vai/nodes/argmax.h:9-18, 57-79; vai/shaders/argmax.comp).  Ties resolve to the
 * lowest index, as torch.argmax (the reference's test oracle) does.  Enqueues one
 * kernel on `stream`; no allocation, no synchronisation. */
VAICU_API int vaicu_argmax_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, void* out_u32);

/* Argmax in two stages, for wide rows and for vocabulary-split heads.  Stage 1 scans
 * column segments of 8192 in parallel blocks, stage 2 folds the per-segment candidates;
 * the result is the same index vaicu_argmax_run returns (lowest index among equal maxima).
 *   logits     [M, N] with a row stride of `ld` elements (ld >= N): a slab of wider rows works
 *   index_base added to every column index: the first vocabulary entry of this GPU's slab
 *   workspace  vaicu_argmax_workspace_bytes(M, N) bytes, 16-byte aligned
 *   out_val    [M] fp32 row maxima, or NULL when only indices are wanted
 *   out_u32    [M] uint32 indices
 * vaicu_argmax_merge_run folds candidates of `groups` slabs: slab g's candidate for row m
 * is vals[g * group_stride + m] / idx[g * group_stride + m] (group_stride >= M, in elements;
 * an all-gather of one [2, M] buffer per GPU gives group_stride = 2 M), so a
 * column-split lm_head exchanges 8 bytes per row and GPU instead of its logits.  This is
 * the sharded form of vAi's Argmax node (vai/nodes/argmax.h:9-18); the reference has no
 * multi-GPU counterpart. */
VAICU_API int vaicu_argmax_workspace_bytes(uint32_t M, uint32_t N, size_t* out_bytes);
VAICU_API int vaicu_argmax_pairs_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, size_t ld,
                                     uint32_t index_base, void* workspace, float* out_val, void* out_u32);
VAICU_API int vaicu_argmax_merge_run(vaicu_stream_t stream, const float* vals, const void* idx_u32, uint32_t groups,
                                     size_t group_stride, uint32_t M, float* out_val, void* out_u32);

/* Top-k sampling over logits [M, N]: vAi's TopKSampling node (vai/nodes/topk-sampling.h:9-31,
 * vai/shaders/topk-sampling.comp): keep the k largest logits of each row ranked by (value
 * descending, index ascending), softmax over them at `temperature` (floored at 1e-6), sample by
 * inverse CDF with the uniform *u_device in [0, 1) — device memory, so that a recorded launch
 * reads each step's value, as the reference reads its host-visible uniform buffer.
 *   k          1 .. 128 (TopKSampling::maxK); k > N uses N
 *   workspace  vaicu_topk_workspace_bytes(M, N, k) bytes (0 for rows of at most 2048 columns)
 *   out_u32    [M] sampled indices
 * VAICU_ERR_TOO_LARGE for rows of more than 256 * 2048 columns. */
VAICU_API int vaicu_topk_workspace_bytes(uint32_t M, uint32_t N, uint32_t k, size_t* out_bytes);
VAICU_API int vaicu_topk_sample_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, uint32_t k,
                                    float temperature, const float* u_device, void* workspace, void* out_u32);

/* TopKSampling over a vocabulary split across GPUs (vai/nodes/topk-sampling.h:33-57 applied in two steps; the
 * reference is single-device).  Step 1 on every GPU: the k best logits of each row of its slab, in rank order
 * (value descending, index ascending), as k (fp32 bits, uint32 index) pairs per row with index_base (the
 * slab's first vocabulary entry) added; a slab narrower than k pads with (lowest float, 0xFFFFFFFF).
 *   logits     [M, N] with a row stride of `ld` elements: a window of wider rows works
 *   workspace  vaicu_topk_workspace_bytes(M, N, k) bytes (0 for rows of at most 2048 columns)
 *   out_pairs  [M, k] pairs, 8-byte aligned
 * The GPUs all-gather their [M, k] lists (8 k bytes per row and GPU instead of logits).  Step 2 on every
 * GPU with the same uniform: merge `groups` lists per row — list g of row m at pairs[g * group_stride + m *
 * list_len], strides in pairs — keep the best k of the union and sample as vaicu_topk_sample_run does.  The
 * token equals the one the single-GPU node draws from the whole row. */
VAICU_API int vaicu_topk_candidates_run(vaicu_stream_t stream, const void* logits, int dtype, uint32_t M, uint32_t N, size_t ld,
                                        uint32_t k, uint32_t index_base, void* workspace, void* out_pairs);
VAICU_API int vaicu_topk_merge_sample_run(vaicu_stream_t stream, const void* pairs, uint32_t groups, size_t group_stride, uint32_t M,
                                          uint32_t list_len, uint32_t k, float temperature, const float* u_device, void* out_u32);

/* Column-split helper for the multi-GPU layout: the desc of rank `rank` of
 * `world` when W's rows (output columns) are split evenly; for gate_fuse the
 * split is per half.  Fills row offsets into W / bias for that rank. No
 * reference counterpart (the reference is single-device). */
VAICU_API int vaicu_linear_shard_desc(const vaicu_linear_desc* full, int rank, int world,
                            vaicu_linear_desc* shard, uint32_t* w_row_begin, uint32_t* w_row_count);

/* Status text (replaces the VAI_ASSERT message, vai/engine/error.h:8-24). */
VAICU_API const char* vaicu_status_string(int status);
/* Text of the last CUDA error seen by this thread (empty string if none). */
VAICU_API const char* vaicu_last_cuda_error(void);
/* Library version: major * 1000 + minor. */
VAICU_API int vaicu_version(void);

#ifdef __cplusplus
}
#endif
#endif /* VAICU_H */
