// Parameters shared by the host planner and the tcgen05 GEMM kernel.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vaicu {

constexpr size_t kTcMaxSmem = 227u * 1024u;   // opt-in shared memory per CTA on sm_100

// How bias / residual are indexed, resolved on the host so the epilogue avoids a
// 64-bit modulo per element (rule: vAi vai/nodes/linear.h:2333-2338).
enum { OPERAND_NONE = 0, OPERAND_PER_COLUMN = 1, OPERAND_FULL = 2, OPERAND_MODULO = 3 };

struct TcParams {
    void* O;
    const void* bias;
    const void* res;
    float* partial;        // non-null: split-K, raw fp32 partials [splits][M][N]
    unsigned int* tile_done;  // non-null (single-CTA kernel, split-K): per-tile count of finished splits; the CTA that
                              // finishes a tile's last split folds the partials and writes O itself.  All zero
                              // between launches.
    int* status;           // device word set to 1 when a bounded wait expired
    uint32_t M, N, K;      // Linear dims; N counts weight rows (2H with gate)
    uint32_t H;            // output columns when gate (N / 2), else N
    uint32_t bn;           // UMMA N
    uint32_t idesc;        // tcgen05 instruction descriptor
    uint32_t tiles_a, tiles_b, num_tiles, group;
    uint32_t kblocks, kb_per_split, splits;
    uint32_t stages, tmem_cols;
    uint32_t wide;         // unswapped kernel only: 256-row tiles (two A boxes, two accumulators)
    uint32_t pair;         // unswapped kernel only: two CTAs (a cluster of 2) share one 256-row tile through cta_group::2
    uint32_t acc_bufs;     // accumulator buffers in TMEM: 2, or 1 when one tile needs all 512 columns
    int32_t o_dtype, b_dtype, epilogue, residual_order, has_bias, has_res, gate;
    int32_t bias_mode, res_mode;
    uint32_t bias_elems, res_elems;
    uint32_t o_aligned16;
    // Output addressing: element (m, j) goes to dst[m * ldo + col0 + j].  A plain run has
    // n_dst = 1, ldo = the output width, col0 = 0; a column-split run writes its slab into
    // up to 8 wider destinations at once (its own and its peers' over NVLink).
    uint32_t ldo, col0, n_dst;
    uint32_t staged;       // CTA-pair kernel: finished tiles go through shared memory so that stores to the
                           // destinations (peers over NVLink) are whole 128-byte row segments
    void* dst[8];
    // Row-parallel run (rs_rows > 0): the outputs are partial sums over this GPU's slice of K, and
    // row m belongs to GPU m / rs_rows, which folds the ranks' partials.  Element (m, j) then goes to
    // dst[m / rs_rows][(rs_slot * rs_rows + m % rs_rows) * ldo + j]: this rank's slab of the owner's staging.
    uint32_t rs_rows, rs_slot;
    // CTA-pair kernel, last (partial) round of tiles: each of the tiles from tail_first on is cut into
    // tail_split column strips of bn / tail_split, one work item each, so that the round keeps more clusters
    // busy for a shorter time (tail_split = 1: off).  idesc_tail is the instruction descriptor of a strip.
    uint32_t tail_first, tail_split, idesc_tail;
    // Swapped kernel over a group of weight tensors that share the activations (q / k / v): the weight
    // tile at which the second / third tensor begins (kNoGroup: a single tensor).  N is the sum of the
    // members' rows; a group always leaves raw partial sums for the group's fold.
    uint32_t grp_t1, grp_t2;
    // Swapped kernel: weight rows per tile (a multiple of 8, at most 128; see plan_tc).
    uint32_t tile_rows;
    // Swapped kernel, split-K folded inside a cluster: cfold = splits = CTAs per cluster, one work item per
    // CTA, the partial sums cross through distributed shared memory and no workspace or second launch is
    // needed (0: off).  For a group, dst[0..2] are the members' outputs.
    uint32_t cfold;
    float scale;
};
constexpr uint32_t kNoGroup = 0xFFFFFFFFu;

// Work item -> tile, K split, column strip and UMMA N of that item.
__host__ __device__ inline void work_item(const TcParams& p, uint32_t w, uint32_t& tile, uint32_t& z, uint32_t& strip, uint32_t& width)
{
    if (p.tail_split > 1u && w >= p.tail_first) {
        const uint32_t r = w - p.tail_first;
        tile = p.tail_first + r / p.tail_split;
        strip = r - (r / p.tail_split) * p.tail_split;
        width = p.bn / p.tail_split;
        z = 0u;
    } else {
        tile = w / p.splits;
        z = w - tile * p.splits;
        strip = 0u;
        width = p.bn;
    }
}
__host__ __device__ inline uint32_t work_items(const TcParams& p)
{
    return p.tail_split > 1u ? p.tail_first + (p.num_tiles - p.tail_first) * p.tail_split : p.num_tiles * p.splits;
}

// Where output row m goes: the destination buffer and the row index inside it.
__host__ __device__ inline void output_row(const TcParams& p, uint32_t m, uint32_t& owner, size_t& row)
{
    if (p.rs_rows) {
        owner = m / p.rs_rows;
        row = (size_t)p.rs_slot * p.rs_rows + (m - owner * p.rs_rows);
    } else {
        owner = 0xFFFFFFFFu;      // every destination takes the row
        row = m;
    }
}

// Tile order: groups of `group` A-tiles (UMMA-M side) sweep all B-tiles before the
// next group starts, so CTAs running at the same time share operand slabs in L2.
__host__ __device__ inline void tile_coords(const TcParams& p, uint32_t tile, uint32_t& ta, uint32_t& tb)
{
    const uint32_t per_group = p.group * p.tiles_b;
    const uint32_t g = tile / per_group;
    const uint32_t first = g * p.group;
    const uint32_t rows = (p.tiles_a - first < p.group) ? p.tiles_a - first : p.group;
    const uint32_t local = tile - g * per_group;
    ta = first + local % rows;
    tb = local / rows;
}

cudaError_t tc_pair_max_clusters(size_t smem, int* clusters);
cudaError_t tc_swap_max_clusters(size_t smem, unsigned cluster, int* clusters);
// One tiny launch whose bounded mbarrier wait is made to run out; sets *status as the GEMM kernels do.
cudaError_t launch_wait_expiry_selftest(int* status, cudaStream_t stream);
// map_b_tail: the weights' map with the strip box of the tail round (CTA-pair kernel with tail_split > 1; else any valid map).
cudaError_t launch_tc_pair_group(const CUtensorMap& map_act, const CUtensorMap* maps_w, const TcParams& p, int grid, size_t smem,
                                 cudaStream_t stream);
cudaError_t launch_tc_gemm_group(const CUtensorMap* maps_w, const CUtensorMap& map_act, const TcParams& p, int grid, size_t smem,
                                 cudaStream_t stream);
cudaError_t launch_tc_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_b_tail, const TcParams& p,
                           bool swap, int grid, size_t smem, cudaStream_t stream);

}  // namespace vaicu
