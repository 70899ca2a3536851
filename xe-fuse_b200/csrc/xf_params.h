// Kernel parameter block shared by the host planner and the device code.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace xf {

enum : int { DT_BF16 = 0, DT_S8 = 1, DT_F32 = 2, DT_S32 = 3 };
enum : int { UN_NONE = 0, UN_GELU, UN_GELU_TANH, UN_SILU, UN_RELU, UN_SIGMOID, UN_EXP };
enum : int { PAIR_NONE = 0, PAIR_SWIGLU, PAIR_GEGLU, PAIR_ROPE, PAIR_SWAP };

// Device status codes written by a bounded wait that gave up (0 = ok).
enum : int {
  DEV_OK = 0,
  DEV_TIMEOUT_PRODUCER_EMPTY = 1,
  DEV_TIMEOUT_MMA_FULL = 2,
  DEV_TIMEOUT_MMA_TMEM_EMPTY = 3,
  DEV_TIMEOUT_EPI_TMEM_FULL = 4,
  DEV_TIMEOUT_SPLIT_PARTIALS = 5,   // a K slice never saw the other slices' partial accumulators
  DEV_TIMEOUT_CLUSTER_EXCHANGE = 6, // cluster split-K: the other K groups' partials never arrived
  DEV_TIMEOUT_EPI_OPERAND = 7,      // the staged epilogue operand of the last tile never landed
};

struct VecArg {
  const void* ptr;
  long long batch_stride;
  float null_default;
  int dtype;    // DT_F32 / DT_BF16
  int enabled;
  int pad_;
};

struct MatArg {
  const void* ptr;
  long long ld;
  long long batch_stride;
  int dtype;    // DT_BF16 / DT_F32
  int enabled;
};

struct EpiParams {
  MatArg residual;
  MatArg aux_store;
  VecArg row_scale;
  VecArg col_scale;
  VecArg bias;
  MatArg cos_sin;
  int cos_sin_period;
  int unary;
  int pair;
  int compact;  // 1: D holds one value per column pair, [M, N/2]
  float* row_sumsq;   // optional [L][ceil(N/32)][M] sums of squares of the final values, or null
};

struct alignas(64) GemmParams {
  CUtensorMap tm_a;   // [L][M][K], box {128 B of K, 128 rows}, 128-B swizzle
  CUtensorMap tm_b;   // [L][K][N], box {128 B of N, KBLK rows}, 128-B swizzle
  CUtensorMap tm_d;   // [L][M][Nout] bf16, box {32 cols, 32 rows}, 64-B swizzle
  CUtensorMap tm_d_peer[7];  // further copies of D (other GPUs' gathered buffers), same geometry
  // Full-matrix epilogue operand of a CTA's LAST tile, fetched by TMA into an idle pipeline stage
  // while that tile's main loop drains (tail_opnd != 0): residual bf16 [L][M][N], box {64 cols,
  // 128 rows}; or the per-head cos_sin table fp32 [L][M][P], box {32 cols, 128 rows}; 128-B swizzle.
  CUtensorMap tm_opnd;
  // The residual again, box {32 columns, 32 rows}, 64-B swizzle: the geometry of a D store.  With
  // res_tma != 0 an epilogue warp TMA-loads the residual of a 32-column slice into the staging
  // buffer its result will leave from, reads its rows there and overwrites them with the result.
  CUtensorMap tm_res;
  // The auxiliary output (acc + residual, bf16 [M,N]) with the geometry of a D store; with
  // aux_tma != 0 a warp's 32 x 32 block of it leaves through a staging buffer and a TMA store.
  CUtensorMap tm_aux;
  int M, N, K, L;
  int tiles_m, tiles_n;    // in units of the cluster tile (128*CTAS rows x BN columns)
  int num_kb;              // ceil(K / KBLK)
  int group_m;             // rasterisation group height in cluster tiles
  int a_batched, b_batched;  // 0: batch stride 0, always use batch coordinate 0
  int a_k_slab;            // >0: A is stored as K slabs of this many elements (third tensor-map mode)
  int l2_hint_a, l2_hint_b;  // L2 policy of the A / B loads: 0 default, 1 evict last, 2 evict first
  void* D;
  void* D_peer[7];         // further destinations of the same output (peer-mapped memory)
  int num_d_peer;          // 0..7
  long long ldd, batch_d;
  int d_dtype;             // DT_BF16 / DT_F32 / DT_S32
  int direct_store;        // 1: plain global stores for D
  int tail_opnd;           // 0 none, 1 residual, 2 cos_sin table: what tm_opnd describes
  int tail_opnd_boxes;     // boxes of 16 KB that make up one CTA tile of that operand
  int res_tma;             // 1: residual slices come through tm_res instead of per-thread global loads
  int aux_tma;             // 1: the auxiliary output leaves through tm_aux instead of per-thread stores
  int diag;                // diagnostics: bit0 skip the TMA loads, bit1 skip the MMAs (results are garbage)
  int* status;             // device status word (may be null)
  // Split-K of the remainder wave: work items [0, split_first) are whole tiles; the tiles from
  // split_first on are each cut into split_s K slices, one work item per slice.  Slices publish
  // raw partial accumulators in split_partials, wait for one another (split_counters), and each
  // sums, in slice order, its share of the tile's columns and runs the epilogue there.
  // split_s == 0: no split.
  int split_first;
  int split_s;
  int total_items;
  int* split_counters;     // [split tiles][CTAS][8]: [0] published, [1] done; zero between launches
  float* split_partials;   // [split tiles][split_s][CTAS][128][BN] raw accumulator words
  long long wait_budget;   // clock64 cycles a wait may take before giving up
  EpiParams epi;
};

}  // namespace xf
