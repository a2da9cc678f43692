// Launch interface of the persistent grouped-GEMM kernel (gemm_sm100.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>
#include <cstdint>

#include "bmoe_b200.h"

namespace bmoe {

// How a CTA obtains its next tile.
enum SchedMode : uint32_t {
  kSchedStatic = 0,  // tile = blockIdx.x + i * gridDim.x
  kSchedQueue = 1,   // global atomic queue (chunked main part + claim-1 tail)
  kSchedClc = 2,     // one CTA per tile, cluster-launch-control work stealing
};

// Where a bounded wait gave up (bmoe_device_report::code).
enum DeviceSite : uint32_t {
  kSiteNone = 0,
  kSiteSchedSlot = 1,     // scheduler waiting for a free tile-info slot
  kSiteSchedPace = 2,     // scheduler waiting for the producer to catch up
  kSiteSchedClc = 3,      // scheduler waiting for a launch-control answer
  kSiteProducerInfo = 4,  // producer waiting for tile info
  kSiteProducerStage = 5, // producer waiting for a free smem stage
  kSiteMmaInfo = 6,
  kSiteMmaAccum = 7,      // MMA waiting for a drained accumulator
  kSiteMmaStage = 8,      // MMA waiting for operand bytes
  kSiteEpiInfo = 9,
  kSiteEpiAccum = 10,     // epilogue waiting for a finished accumulator
  kSiteSchedGate = 11,    // scheduler waiting for another rank's rows (stage = group, aux = rank)
  kSiteExpandFlag = 12,   // row expansion waiting for a source's flag (stage = group, aux = rank)
  kSiteSchedExpand = 13,  // scheduler waiting for a group's row expansion (stage = group)
  kSiteCheck = 14,        // -DBMOE_CHECKS build: a tile record failed a bounds check
                          // (stage = DeviceCheck, aux = the offending value)
};

// What a -DBMOE_CHECKS build verifies for every tile record before publishing it to the
// roles (everything the TMA coordinates, descriptor indices and Tensor Memory columns of the
// tile derive from). A failure is reported through DeviceStatus and ends the launch through
// the abort path of the bounded waits; nothing traps.
enum DeviceCheck : uint32_t {
  kCheckTileIndex = 1,   // worklist index >= tile total
  kCheckExpert = 2,      // expert id >= experts (indexes the descriptor arrays)
  kCheckColumns = 3,     // col0 / valid_n outside [0, n] or wider than the tile
  kCheckRows = 4,        // valid_m outside [1, tile rows]
  kCheckPackedRows = 5,  // packed A: rows beyond the buffer
  kCheckKBlocks = 6,     // k-blocks do not cover k (TMA x coordinate = multiples of 128 B)
  kCheckTmemColumns = 7, // accumulator buffers exceed the allocated Tensor Memory columns
};

// Device-side error record; zero-initialised by the host.
struct DeviceStatus {
  uint32_t count;  // number of reports (first one owns the fields below)
  uint32_t code;
  uint32_t cta;
  uint32_t role;
  uint32_t tile;
  uint32_t stage;
  uint32_t aux;
  uint32_t reserved;
};

struct GemmParams {
  const CUtensorMap* tmap_a;  // [experts] A_e as {k, M_e}, box {128 B, a_box_bytes / 128}
  const CUtensorMap* tmap_b;  // [experts] B_e as {k, n},   box {128 B, TILE_N / cta_group}
  const CUtensorMap* tmap_d;  // [experts] D_e as {n, M_e}, box {64, 32} BF16 / {32, 32} FP32
  const bmoe_tile* tiles;     // device worklist
  uint32_t tile_count;
  uint32_t k_blocks;          // ceil(k bytes of a row / 128)
  uint32_t sched_mode;        // SchedMode
  uint32_t claim_size;        // queue: tiles per claim in the main part
  uint32_t main_end;          // queue: [0, main_end) chunked, [main_end, T) singly
  uint32_t lookahead;         // queue/clc: claims allowed ahead of the producer
  uint32_t* queue;            // [0] main head, [1] tail head, [2] exited CTAs
  DeviceStatus* status;
  uint32_t* tile_visits;      // optional [tile_count]
  uint32_t* cta_tiles;        // optional [gridDim.x]
  uint64_t* trace;            // optional [gridDim.x][kTraceWords] wait accounting
  uint64_t wait_budget_ns;
  // Optional gate (expert-parallel exchange): a tile of expert e is published only
  // after flag slots gate_group_of[e] * gate_ranks + r (r != gate_self) reached
  // gate_epoch. The flags are raised by OTHER GPUs when their rows have landed.
  const uint32_t* gate_flags;   // nullptr = no gate
  const uint8_t* gate_group_of; // [experts]
  uint32_t gate_epoch;
  uint32_t gate_ranks;
  uint32_t gate_self;
  // Rows that arrive as peer copies have a flag plane of their own behind the first one
  // (gate_copy_plane slots further): group g also waits for the sources whose bit is set
  // in gate_copy_mask[g]. nullptr = no such rows.
  const uint32_t* gate_copy_mask;
  uint32_t gate_copy_plane;
  // Optional result push (expert-parallel exchange, BF16 output): instead of the TMA
  // store into D, the epilogue writes every valid tile row to row `assignment` of its
  // origin rank's result buffer (plain 16-byte stores, 128 contiguous bytes per row
  // and chunk; peer memory over NVLink or local memory).
  const long long* push_origin;     // [packed rows] rank << 40 | assignment; nullptr = off
  const uint32_t* push_expert_row;  // [experts] first packed row of each expert
  uint4* const* push_bases;         // [push_ranks] result buffers
  uint64_t push_rows_cap;           // rows each result buffer holds
  uint32_t push_vec_per_row;        // n / 8
  uint32_t push_ranks;
  // Optional packed A: when non-null, tmap_a[0] describes ONE row-major buffer that
  // holds the rows of all experts back to back and a_row_offsets[e] is the first row of
  // expert e in it (the worklist builder's row-offset array). A tile at an expert's
  // ragged edge then also loads rows of the next expert; they only feed accumulator
  // rows beyond valid_m, which are never written.
  const unsigned long long* a_row_offsets;
  // Optional: the tile total lives in device memory (written by the worklist builder of
  // the same stream; the host never saw the counts). tile_count is then only the
  // capacity of `tiles`, and the queue's chunked part ends at the tile total.
  const uint32_t* tile_count_dev;
  // Optional row expansion (send-once exchange): record lists {from row, to row} per
  // (exchange group, source rank), written by the sources. Warp 3 of every CTA copies
  // A[from] -> A[to] for a list once that source's flag for the group is up; the gate
  // waits until expand_done[group] has reached the sum of the group's list lengths.
  const uint2* expand_records;    // [groups][gate_ranks][expand_cap]; nullptr = off
  const uint32_t* expand_count;   // [groups][gate_ranks] list lengths (valid once flagged)
  uint32_t* expand_next;          // [groups][gate_ranks] claim counters, zero at step start
  uint32_t* expand_done;          // [groups] records carried out, zero at step start
  uint4* expand_a;                // packed A
  uint64_t expand_rows_cap;
  uint32_t expand_vec_per_row;    // k / 8
  uint32_t expand_cap;
  uint32_t expand_groups;
  // Bytes of one A box: rows of the box x 128. 128 rows unless no expert has that many:
  // then the box only covers the rows that can be valid (rounded up to 8). The MMA still
  // reads 128 rows of the stage; the rows the box does not write feed accumulator rows
  // that are never stored. What it saves is shared-memory fill bandwidth: a CTA takes in
  // about 64 bytes per cycle, zero-filled rows included, and that - not HBM or the tensor
  // pipe - bounds a one-wave launch over a small-M problem.
  uint32_t a_box_bytes;
  // Operand type: 0 = BF16 (k-block = 64 elements, kind::f16), 1 = FP8 E4M3 (k-block =
  // 128 elements, kind::f8f6f4). A k-block is 128 bytes of a row either way and one MMA
  // instruction covers 32 of them, so the shared-memory layout, the descriptors and the
  // pipeline are the same; only the tensor maps, k_blocks and the instruction differ.
  uint32_t fp8;
  // Extents for the -DBMOE_CHECKS build (always filled in by the plan, read by that build only).
  uint32_t check_experts;
  uint32_t check_n;
  uint32_t check_k_bytes;     // bytes of an operand row
  uint64_t check_a_rows;      // rows of the packed A buffer (0 = per-expert A maps)
};

// Words per CTA of GemmParams::trace (SM cycles):
//   0 producer waiting for tile info      1 producer waiting for a free stage
//   2 MMA waiting for tile info           3 MMA waiting for a drained accumulator
//   4 MMA waiting for operand bytes       5 epilogue waiting for tile info
//   6 epilogue waiting for an accumulator 7 epilogue draining (ld, convert, store)
//   8 tiles run by this CTA               9 kernel cycles of this CTA
//   10 MMA lane issuing tcgen05.mma / commit
// and a time line of the CTA, in cycles since its first instruction:
//   11 set-up done (barriers, Tensor Memory)   12 first operand stage landed
//   13 last MMA of the last tile issued         14 last accumulator complete
//   15 epilogue done (stores of the last tile issued and drained)
constexpr uint32_t kTraceWords = 16;

// Dynamic shared memory / operand stages for a tile width (64, 128 or 256) and CTA
// group (1 = single CTA, 2 = CTA pair computing 256-row tiles; needs tile_n 256).
uint32_t gemm_smem_bytes(uint32_t tile_n, uint32_t cta_group);
uint32_t gemm_stage_count(uint32_t tile_n, uint32_t cta_group);

// Enqueues the kernel on `units` scheduling units: persistent CTAs (or CTA
// pairs), or the tile count for CLC. The grid is units * cta_group CTAs.
// out_f32 selects the FP32-output epilogue (tile_n 256 only).
cudaError_t launch_grouped_gemm(const GemmParams& params, uint32_t tile_n,
                                uint32_t cta_group, bool out_f32, uint32_t units,
                                cudaStream_t stream);

}  // namespace bmoe
