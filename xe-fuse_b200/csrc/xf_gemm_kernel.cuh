// Persistent, warp-specialised fused GEMM + epilogue kernel for sm_100a.
//
//   D = epilogue(A[M,K] * B[K,N])      A row-major (K contiguous), B row-major (N contiguous)
//
// One CTA (CTAS == 1) or a pair of CTAs on neighbouring SMs (CTAS == 2, cta_group::2) owns a
// (128*CTAS) x BN output tile.  Roles inside a 384-thread CTA:
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the A and B stages
//   warp 1      MMA issuer:   one lane issues tcgen05.mma (kind::f16 / kind::i8) into TMEM
//   warp 2      TMEM allocator
//   warps 4-11  epilogue, two warps per TMEM lane quadrant taking alternate 32-column units:
//               tcgen05.ld the accumulator (one row per thread, 32 columns per load), run the flat
//               epilogue program in registers, stage bf16 rows in swizzled shared memory and
//               TMA-store them; warps 0-3 join them for the CTA's last tile
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps
// the main loop of tile i+1.  Adjacent output columns (2k, 2k+1) are adjacent registers of one
// thread, so SwiGLU / GeGLU / RoPE need no cross-lane traffic.
//
// Work items are whole tiles, except that the tiles of a partly filled last wave may be cut into K
// slices (GemmParams::split_s): the slices exchange raw accumulators through global memory and
// share the finishing work (see the epilogue role).
//
// Small problems (at most one 256 x 256 tile per four SMs) use the cluster split-K variants
// (KC == 2): a cluster holds KC CTA pairs that each accumulate one K range of the SAME tile into
// their own TMEM; the pairs then swap partial accumulators through distributed shared memory
// (st.shared::cluster into the partner's idle pipeline stages) and each pair finishes BN / KC of the
// tile's columns.  No global scratch, no second launch.
//
// Every tile variant is compiled once per epilogue class (template parameter EM, a mask of EF_*
// features): the flat epilogue program is read at run time, but an instance only carries the code
// of the steps its mask names; the host launches the smallest class that covers a descriptor.
//
// Shared memory per stage: A 128 rows x 128 B (K-major, 128-B swizzle) and B as BN/CTAS columns
// split into 128-B column groups of KBLK rows each (MN-major, 128-B swizzle), exactly as the TMA
// boxes land.  With CTAS == 2 each CTA loads its own 128 rows of A and its own half of the B
// columns; no load is multicast.
#pragma once

#include <cuda_bf16.h>

#include "xf_params.h"
#include "xf_ptx.cuh"

namespace xf {

template <int KIND, int BN_, int CTAS_, int KS_, int KC_ = 1>
struct TileCfg {
  static constexpr int BN = BN_;
  static constexpr int CTAS = CTAS_;
  static constexpr int KS = KS_;                       // 128-byte K slabs per pipeline stage
  static constexpr int KC = KC_;                       // CTA pairs of a cluster that share one tile's K range
  static constexpr int CLUSTER = CTAS_ * KC_;          // CTAs per cluster
  static constexpr int BM = 128;                       // rows per CTA
  static constexpr int ES = (KIND == 0) ? 2 : 1;       // bytes per A/B element
  static constexpr int KSLAB = 128 / ES;               // K elements in one 128-byte slab
  static constexpr int KBLK = KS * KSLAB;              // K elements per stage
  static constexpr int UK = 32 / ES;                   // K elements per tcgen05.mma
  static constexpr int BN_CTA = BN / CTAS;             // B columns one CTA loads
  static constexpr int GRP_COLS = 128 / ES;            // columns per 128-B group
  static constexpr int NGRP = BN_CTA / GRP_COLS;       // column groups per CTA
  static constexpr int GRP_BYTES = KBLK * 128;         // one column group: KBLK rows of 128 B
  static constexpr int A_SLAB_BYTES = BM * 128;        // 128 rows x 128 B of K
  static constexpr int A_BYTES = KS * A_SLAB_BYTES;
  static constexpr int B_BYTES = NGRP * GRP_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF_BYTES = 2048;           // 32 rows x 64 B
  static constexpr int EPI_WARPS = 8;                  // two per TMEM lane quadrant
  static constexpr int THREADS = (4 + EPI_WARPS) * 32;
  static constexpr int EPI_BUFS = 2;                   // staging buffers per epilogue warp
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUFS * EPI_BUF_BYTES;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_LIMIT = 227 * 1024;
  static constexpr int STAGES_RAW =
      (SMEM_LIMIT - 1024 - EPI_BYTES - BAR_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES =
      1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;             // double-buffered accumulator
  // Cluster split-K: the pipeline stage the MMAs leave first receives the other K groups' partial
  // accumulators of the columns this CTA finishes: (KC-1) x 128 rows x BN/KC columns x 4 B.
  static constexpr int XCHG_SLICES = BN / KC / 32;     // 32-column accumulator slices per K group
  static constexpr int XCHG_BYTES = (KC - 1) * BM * (BN / KC) * 4;
  static_assert(KC == 1 || (CTAS == 2 && BN == 256), "cluster split-K is built for paired 256-column tiles");
  static_assert(KC == 1 || (XCHG_BYTES <= STAGE_BYTES && STAGES >= 3), "exchange buffer exceeds a stage");
  static_assert(NGRP >= 1, "B tile narrower than one 128-byte column group");
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512 || TMEM_COLS == 128, "TMEM columns");
  static_assert(STAGES >= 2, "not enough shared memory for a pipeline");
};

// tcgen05 instruction descriptor: D format, A/B formats, A K-major, B MN-major, N>>3, M>>4.
template <int KIND, int BN, int CTAS>
__host__ __device__ constexpr uint32_t make_idesc() {
  uint32_t c_fmt = (KIND == 0) ? 1u : 2u;  // F32 : S32
  uint32_t ab_fmt = 1u;                    // BF16 (kind::f16) : signed 8-bit (kind::i8)
  return (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | (0u << 15) | (1u << 16) |
         (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>((128 * CTAS) >> 4) << 24);
}

struct TileCoord {
  int tm, tn, l;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int tile) {
  TileCoord c;
  const int per_batch = p.tiles_m * p.tiles_n;
  c.l = tile / per_batch;
  const int r = tile - c.l * per_batch;
  const int grp_tiles = p.group_m * p.tiles_n;
  const int grp = r / grp_tiles;
  const int first_m = grp * p.group_m;
  const int gsz = min(p.group_m, p.tiles_m - first_m);
  const int rr = r - grp * grp_tiles;
  c.tn = rr / gsz;
  c.tm = first_m + (rr - c.tn * gsz);
  return c;
}

// One unit of the persistent schedule: a whole tile, or one K slice of a split tile.
struct WorkItem {
  int tile, kb0, kb1, slice, split_idx;   // split_idx < 0: whole tile
};

// Order in which a scheduling unit takes its work items.  Unit u owns items u, u + U, u + 2U, ...;
// whole tiles come first in that numbering and a K slice, if the unit has one, last (item
// split_first + u, split_first being a multiple of U).  The unit runs its slice FIRST: all slices
// of a tile then start together when the kernel starts, and their exchange through global memory
// (publish, wait, sum) hides behind the main loop of the unit's next tile instead of trailing the
// kernel.  Maps the loop variable w (u, u + U, ...) to the item to run.
__device__ __forceinline__ int schedule_item(const GemmParams& p, int w, int unit, int num_units) {
  if (p.split_s == 0 || unit >= p.total_items - p.split_first || p.split_first == 0) return w;
  return (w == unit) ? p.split_first + unit : w - num_units;
}

__device__ __forceinline__ WorkItem decode_item(const GemmParams& p, int w) {
  WorkItem it;
  if (p.split_s == 0 || w < p.split_first) {
    it.tile = w; it.kb0 = 0; it.kb1 = p.num_kb; it.slice = 0; it.split_idx = -1;
  } else {
    const int j = w - p.split_first;
    it.split_idx = j / p.split_s;
    it.slice = j - it.split_idx * p.split_s;
    it.tile = p.split_first + it.split_idx;
    it.kb0 = static_cast<int>(static_cast<long long>(it.slice) * p.num_kb / p.split_s);
    it.kb1 = static_cast<int>(static_cast<long long>(it.slice + 1) * p.num_kb / p.split_s);
  }
  return it;
}

__device__ __forceinline__ float load_vec_elem(const VecArg& v, long long idx) {
  if (v.ptr == nullptr) return v.null_default;
  if (v.dtype == DT_BF16)
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(v.ptr)[idx]);
  return reinterpret_cast<const float*>(v.ptr)[idx];
}

// 32 consecutive elements of a per-column vector starting at column col0 (every lane of a warp
// reads the same addresses: one L1 transaction per load).  Columns >= n_total read as `fill`.
__device__ __forceinline__ void load_vec32(const VecArg& a, int l, int col0, int n_total, float fill,
                                           float (&out)[32]) {
  if (a.ptr == nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = a.null_default;
    return;
  }
  const long long off = static_cast<long long>(l) * a.batch_stride + col0;
  if (a.dtype == DT_BF16) {
    const __nv_bfloat16* ptr = reinterpret_cast<const __nv_bfloat16*>(a.ptr) + off;
    if (col0 + 32 <= n_total && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(ptr) + j);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          out[j * 8 + t * 2 + 0] = __uint_as_float(w[t] << 16);
          out[j * 8 + t * 2 + 1] = __uint_as_float(w[t] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = (col0 + i < n_total) ? __bfloat162float(ptr[i]) : fill;
    }
  } else {
    const float* ptr = reinterpret_cast<const float*>(a.ptr) + off;
    if (col0 + 32 <= n_total && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(ptr) + j);
        out[j * 4 + 0] = f.x; out[j * 4 + 1] = f.y; out[j * 4 + 2] = f.z; out[j * 4 + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = (col0 + i < n_total) ? ptr[i] : fill;
    }
  }
}

// v[i] = v[i] * a[col0 + i] (MUL) or v[i] + a[col0 + i] over 32 consecutive elements of a per-column
// vector, consumed 16 bytes at a time so no 32-element temporary is alive beside v.  Every lane of a
// warp reads the same addresses (one L1 transaction per load); columns >= n_total count as `fill`.
template <bool MUL>
__device__ __forceinline__ void apply_vec32(const VecArg& a, int l, int col0, int n_total, float fill,
                                            float (&v)[32]) {
  auto op = [](float x, float y) { return MUL ? x * y : x + y; };
  if (a.ptr == nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = op(v[i], a.null_default);
    return;
  }
  const long long off = static_cast<long long>(l) * a.batch_stride + col0;
  if (a.dtype == DT_BF16) {
    const __nv_bfloat16* ptr = reinterpret_cast<const __nv_bfloat16*>(a.ptr) + off;
    if (col0 + 32 <= n_total && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(ptr) + j);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          v[j * 8 + t * 2 + 0] = op(v[j * 8 + t * 2 + 0], __uint_as_float(w[t] << 16));
          v[j * 8 + t * 2 + 1] = op(v[j * 8 + t * 2 + 1], __uint_as_float(w[t] & 0xFFFF0000u));
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = op(v[i], (col0 + i < n_total) ? __bfloat162float(ptr[i]) : fill);
    }
  } else {
    const float* ptr = reinterpret_cast<const float*>(a.ptr) + off;
    if (col0 + 32 <= n_total && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(ptr) + j);
        v[j * 4 + 0] = op(v[j * 4 + 0], f.x); v[j * 4 + 1] = op(v[j * 4 + 1], f.y);
        v[j * 4 + 2] = op(v[j * 4 + 2], f.z); v[j * 4 + 3] = op(v[j * 4 + 3], f.w);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = op(v[i], (col0 + i < n_total) ? ptr[i] : fill);
    }
  }
}

__device__ __forceinline__ float unary_apply(int op, float x) {
  switch (op) {
    case UN_GELU: return x * 0.5f * (1.0f + erff(x * 0.7071067811865475f));
    case UN_GELU_TANH: {
      const float k = 0.7978845608028654f;
      float x3 = x * x * x;
      return x * 0.5f * (1.0f + tanhf(k * (x + 0.044715f * x3)));
    }
    case UN_SILU: return __fdividef(x, 1.0f + __expf(-x));
    case UN_RELU: return x > 0.0f ? x : 0.0f;
    case UN_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-x));
    case UN_EXP: return __expf(x);
    default: return x;
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // .x = lo (low 16 bits), .y = hi
  return *reinterpret_cast<uint32_t*>(&h);
}

// Reading 32 consecutive elements of row `row` of a full [M,N] operand (residual, cos_sin) as floats,
// in two phases so the loads can be in flight while the accumulator is read out of TMEM.
// Phase 1 issues the 16-byte loads into raw words (bf16 uses raw[0..3], fp32 raw[0..7]) and returns
//   1: loads issued   2: ragged or unaligned, phase 2 reads element by element.
__device__ __forceinline__ int mat_row32_issue(const MatArg& m, int l, int row, int col0,
                                               int ncols_total, uint4 (&raw)[8]) {
  const long long off = static_cast<long long>(l) * m.batch_stride +
                        static_cast<long long>(row) * m.ld + col0;
  if (m.dtype == DT_BF16) {
    const __nv_bfloat16* ptr = reinterpret_cast<const __nv_bfloat16*>(m.ptr) + off;
    if (col0 + 32 <= ncols_total && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) raw[j] = __ldg(reinterpret_cast<const uint4*>(ptr) + j);
      return 1;
    }
    return 2;
  }
  const float* ptr = reinterpret_cast<const float*>(m.ptr) + off;
  if (col0 + 32 <= ncols_total && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) raw[j] = __ldg(reinterpret_cast<const uint4*>(ptr) + j);
    return 1;
  }
  return 2;
}

// Phase 2: decodes the raw words (mode 1) or reads the elements one by one (mode 2).  Columns >=
// ncols_total read as 0.
__device__ __forceinline__ void mat_row32_finish(int mode, const uint4 (&raw)[8], const MatArg& m,
                                                 int l, int row, int col0, int ncols_total,
                                                 float (&out)[32]) {
  if (mode == 1) {
    if (m.dtype == DT_BF16) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          out[j * 8 + t * 2 + 0] = __uint_as_float(w[t] << 16);
          out[j * 8 + t * 2 + 1] = __uint_as_float(w[t] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        out[j * 4 + 0] = __uint_as_float(raw[j].x); out[j * 4 + 1] = __uint_as_float(raw[j].y);
        out[j * 4 + 2] = __uint_as_float(raw[j].z); out[j * 4 + 3] = __uint_as_float(raw[j].w);
      }
    }
    return;
  }
  const long long off = static_cast<long long>(l) * m.batch_stride +
                        static_cast<long long>(row) * m.ld + col0;
  if (m.dtype == DT_BF16) {
    const __nv_bfloat16* ptr = reinterpret_cast<const __nv_bfloat16*>(m.ptr) + off;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      out[i] = (col0 + i < ncols_total) ? __bfloat162float(ptr[i]) : 0.0f;
  } else {
    const float* ptr = reinterpret_cast<const float*>(m.ptr) + off;
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = (col0 + i < ncols_total) ? ptr[i] : 0.0f;
  }
}

__device__ __forceinline__ void load_mat_row32(const MatArg& m, int l, int row, int col0,
                                               int ncols_total, float (&out)[32]) {
  uint4 raw[8];
  const int mode = mat_row32_issue(m, l, row, col0, ncols_total, raw);
  mat_row32_finish(mode, raw, m, l, row, col0, ncols_total, out);
}

// The same 32 elements out of an operand tile that TMA staged in shared memory: boxes of 128 rows x
// 128 bytes (64 bf16 or 32 fp32 columns) with the 128-byte swizzle, one after the other.  `col` is
// the column inside the staged tile (a multiple of 32), `r` the row inside the CTA tile.  Eight
// consecutive lanes read eight different 16-byte positions, so the loads are conflict-free.
__device__ __forceinline__ void mat_row32_from_smem(const uint8_t* tile, bool bf16, int r, int col,
                                                    uint4 (&raw)[8]) {
  if (bf16) {
    const uint8_t* row = tile + (col >> 6) * 16384 + r * 128;
    const int c0 = (col & 63) >> 3;          // first 16-byte chunk of the 32 columns inside the 128-byte row
#pragma unroll
    for (int j = 0; j < 4; ++j)
      raw[j] = *reinterpret_cast<const uint4*>(row + (((c0 + j) ^ (r & 7)) << 4));
  } else {
    const uint8_t* row = tile + (col >> 5) * 16384 + r * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      raw[j] = *reinterpret_cast<const uint4*>(row + ((j ^ (r & 7)) << 4));
  }
}

// Column of the cos_sin operand that output column gcol reads, and the operand's width.
__device__ __forceinline__ int cos_sin_col(const EpiParams& e, int gcol) {
  return e.cos_sin_period > 0 ? (gcol % e.cos_sin_period) : gcol;
}
__device__ __forceinline__ int cos_sin_width(const EpiParams& e, int N) {
  return e.cos_sin_period > 0 ? e.cos_sin_period : N;
}

// Epilogue features a kernel instance is COMPILED with (template parameter EM).  The flat program is
// still read at run time, but an instance only carries the code of the steps its mask names: the
// epilogue of a CTA's last tile runs with nothing to hide behind, a few times per warp, and every
// taken branch over code that is never executed costs it an instruction fetch from far away (a
// minimal epilogue took 0.35 us less per 32-column slice than the all-in-one one).  The host picks
// the smallest instance that covers a descriptor; row scale, column scale and bias are in all of them.
enum : int {
  EF_MAT = 1,     // full-matrix residual and the auxiliary (dual) output
  EF_UNARY = 2,   // GeLU / SiLU / ... element-wise activations
  EF_GLU = 4,     // SwiGLU / GeGLU pairs, also the compact [M, N/2] layout
  EF_ROPE = 8,    // rotary pairs with a cos_sin operand
  EF_MISC = 16,   // pair swap, fp32 / int32 outputs, per-thread (non-TMA) stores, row_sumsq side output
  EF_ALL = 31
};

// Which full-matrix operand of the flat program is fetched ahead of the accumulator read.
enum : int { PRE_NONE = 0, PRE_RESIDUAL = 1, PRE_COS_SIN = 2 };
template <int EM>
__device__ __forceinline__ int preload_choice(const EpiParams& e) {
  if constexpr ((EM & EF_ROPE) != 0) {
    if (e.pair == PAIR_ROPE) return PRE_COS_SIN;
  }
  if constexpr ((EM & EF_MAT) != 0) {
    if (e.residual.enabled) return PRE_RESIDUAL;
  }
  return PRE_NONE;
}

// Asks L2 for this row's part of the full-matrix operands of tile columns [n0, n0 + ncols): issued
// by the epilogue warps while the tile's main loop still runs, so the operand reads of the epilogue
// proper hit L2 instead of waiting for HBM.  `part` of `nparts` warps that share the row.
template <int EM>
__device__ __forceinline__ void prefetch_tile_operands(const EpiParams& e, int N, int l, int row,
                                                       int n0, int ncols, int part, int nparts) {
  if ((EM & EF_MAT) && e.residual.enabled) {
    const int es = e.residual.dtype == DT_BF16 ? 2 : 4;
    const char* base = reinterpret_cast<const char*>(e.residual.ptr) +
                       (static_cast<long long>(l) * e.residual.batch_stride +
                        static_cast<long long>(row) * e.residual.ld + n0) * es;
    for (int off = part * 128; off < ncols * es; off += nparts * 128) ptx::prefetch_l2(base + off);
  }
  if ((EM & EF_ROPE) && e.pair == PAIR_ROPE) {
    const int width = cos_sin_width(e, N);
    int c0 = cos_sin_col(e, n0), nc = ncols;
    if (nc >= width) { c0 = 0; nc = width; }          // the tile walks the whole per-head table
    if (c0 + nc > width) nc = width - c0;
    const char* base = reinterpret_cast<const char*>(e.cos_sin.ptr) +
                       (static_cast<long long>(l) * e.cos_sin.batch_stride +
                        static_cast<long long>(row) * e.cos_sin.ld + c0) * 4;
    for (int off = part * 128; off < nc * 4; off += nparts * 128) ptx::prefetch_l2(base + off);
  }
}

// Stores `n` (<= 32) packed bf16 values (pk holds pairs) to row-major global memory.
__device__ __forceinline__ void store_bf16_row(__nv_bfloat16* ptr, const uint32_t* pk, int nvalid,
                                               int nfull) {
  if (nvalid >= nfull && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
    uint4* p4 = reinterpret_cast<uint4*>(ptr);
    for (int j = 0; j < nfull / 8; ++j)
      p4[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
  } else {
    for (int i = 0; i < nfull; ++i) {
      if (i < nvalid) {
        uint32_t w = pk[i >> 1];
        uint16_t h = (i & 1) ? static_cast<uint16_t>(w >> 16) : static_cast<uint16_t>(w & 0xFFFF);
        reinterpret_cast<uint16_t*>(ptr)[i] = h;
      }
    }
  }
}

// Runs the flat epilogue program on 32 accumulator columns of one row.
//   r      raw TMEM words (fp32 bits or int32)
//   v      results; for the compact layout only v[0..15] are meaningful (one per pair)
//   gcol0  global column of r[0]
//   pre_which / pre_mode / pre   the full-matrix operand whose loads were issued ahead of the
//          accumulator read (mat_row32_issue), if any; the other one is loaded here
//   staged / srow / scol   the operand tile TMA staged in shared memory for a CTA's last tile (or
//          null), this thread's row in it and the first of the 32 columns; it takes the place of
//          `pre`, whose registers then carry the next accumulator slice
//   aux_row / aux_sw   non-null: the auxiliary output of this row goes to these 64 bytes of a
//          64-byte-swizzled staging buffer (16-byte chunk j at (j ^ aux_sw)) and the caller stores
//          the buffer with TMA; null: the thread stores its row to global memory itself
__device__ __forceinline__ void rope_pair(float xe, float xo, float c, float s, float& oe, float& oo) {
  oe = xe * c + xo * s;
  oo = -xe * s + xo * c;
}

template <int KIND, int EM>
__device__ __forceinline__ void epilogue_chunk(const EpiParams& e, int N, const uint32_t (&r)[32],
                                               float (&v)[32], int row, bool row_ok, int l,
                                               int gcol0, float rs, int pre_which, int pre_mode,
                                               const uint4 (&pre)[8], const uint8_t* staged, int srow,
                                               int scol, uint8_t* aux_row = nullptr, int aux_sw = 0) {
#pragma unroll
  for (int i = 0; i < 32; ++i)
    v[i] = (KIND == 0) ? __uint_as_float(r[i]) : static_cast<float>(static_cast<int>(r[i]));

  if constexpr ((EM & EF_MAT) != 0) {
  if (e.residual.enabled && row_ok) {
    if (staged != nullptr && pre_which == PRE_RESIDUAL) {
      const uint8_t* srow_ptr = staged + (scol >> 6) * 16384 + srow * 128;
      const int c0 = (scol & 63) >> 3;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 x = *reinterpret_cast<const uint4*>(srow_ptr + (((c0 + j) ^ (srow & 7)) << 4));
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          v[j * 8 + t * 2 + 0] += __uint_as_float(w[t] << 16);
          v[j * 8 + t * 2 + 1] += __uint_as_float(w[t] & 0xFFFF0000u);
        }
      }
    } else if (pre_which == PRE_RESIDUAL && pre_mode == 1 && e.residual.dtype == DT_BF16) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {     // the words requested ahead of the accumulator read
        const uint32_t w[4] = {pre[j].x, pre[j].y, pre[j].z, pre[j].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          v[j * 8 + t * 2 + 0] += __uint_as_float(w[t] << 16);
          v[j * 8 + t * 2 + 1] += __uint_as_float(w[t] & 0xFFFF0000u);
        }
      }
    } else {
      float t[32];
      if (pre_which == PRE_RESIDUAL) mat_row32_finish(pre_mode, pre, e.residual, l, row, gcol0, N, t);
      else load_mat_row32(e.residual, l, row, gcol0, N, t);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += t[i];
    }
  }
  if (e.aux_store.enabled && row_ok) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
    if (aux_row != nullptr) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(aux_row + ((j ^ aux_sw) << 4)) =
            make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    } else {
      __nv_bfloat16* ptr = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(e.aux_store.ptr)) +
                           static_cast<long long>(l) * e.aux_store.batch_stride +
                           static_cast<long long>(row) * e.aux_store.ld + gcol0;
      store_bf16_row(ptr, pk, N - gcol0, 32);
    }
  }
  }   // EF_MAT
  if (e.row_scale.enabled) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= rs;
  }
  if (e.col_scale.enabled) apply_vec32<true>(e.col_scale, l, gcol0, N, 1.0f, v);
  if (e.bias.enabled) apply_vec32<false>(e.bias, l, gcol0, N, 0.0f, v);
  // The op switches sit OUTSIDE the element loops: every loop body is straight-line code, so the
  // 32 independent elements of a chunk interleave instead of running as one dependent chain each.
  if constexpr ((EM & EF_UNARY) != 0) {
  switch (e.unary) {
    case UN_NONE: break;
#define XF_UNARY_CASE(OP)                                      \
    case OP:                                                   \
      _Pragma("unroll") for (int i = 0; i < 32; ++i) v[i] = unary_apply(OP, v[i]); \
      break;
    XF_UNARY_CASE(UN_GELU)
    XF_UNARY_CASE(UN_GELU_TANH)
    XF_UNARY_CASE(UN_SILU)
    XF_UNARY_CASE(UN_RELU)
    XF_UNARY_CASE(UN_SIGMOID)
    XF_UNARY_CASE(UN_EXP)
#undef XF_UNARY_CASE
    default: break;
  }
  }   // EF_UNARY
  if ((EM & EF_GLU) && (e.pair == PAIR_SWIGLU || e.pair == PAIR_GEGLU)) {
    float o[16];
    if (e.pair == PAIR_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        o[j] = __fdividef(v[2 * j], 1.0f + __expf(-v[2 * j])) * v[2 * j + 1];
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        o[j] = v[2 * j] * 0.5f * (1.0f + erff(v[2 * j] * 0.7071067811865475f)) * v[2 * j + 1];
    }
    if (e.compact) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = o[j];
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) { v[2 * j] = o[j]; v[2 * j + 1] = o[j]; }
    }
  } else if ((EM & EF_ROPE) && e.pair == PAIR_ROPE) {
    if (staged != nullptr && pre_which == PRE_COS_SIN && row_ok) {
      const uint8_t* srow_ptr = staged + (scol >> 5) * 16384 + srow * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 x = *reinterpret_cast<const uint4*>(srow_ptr + ((j ^ (srow & 7)) << 4));
        rope_pair(v[4 * j], v[4 * j + 1], __uint_as_float(x.x), __uint_as_float(x.y), v[4 * j], v[4 * j + 1]);
        rope_pair(v[4 * j + 2], v[4 * j + 3], __uint_as_float(x.z), __uint_as_float(x.w), v[4 * j + 2],
                  v[4 * j + 3]);
      }
    } else if (pre_which == PRE_COS_SIN && pre_mode == 1 && row_ok) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {     // the words requested ahead of the accumulator read
        rope_pair(v[4 * j], v[4 * j + 1], __uint_as_float(pre[j].x), __uint_as_float(pre[j].y), v[4 * j],
                  v[4 * j + 1]);
        rope_pair(v[4 * j + 2], v[4 * j + 3], __uint_as_float(pre[j].z), __uint_as_float(pre[j].w),
                  v[4 * j + 2], v[4 * j + 3]);
      }
    } else {
      float cs[32];
      if (row_ok) {
        const int ccol = cos_sin_col(e, gcol0);
        const int climit = cos_sin_width(e, N);
        if (pre_which == PRE_COS_SIN) mat_row32_finish(pre_mode, pre, e.cos_sin, l, row, ccol, climit, cs);
        else load_mat_row32(e.cos_sin, l, row, ccol, climit, cs);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) cs[i] = 0.0f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) rope_pair(v[2 * j], v[2 * j + 1], cs[2 * j], cs[2 * j + 1], v[2 * j], v[2 * j + 1]);
    }
  } else if ((EM & EF_MISC) && e.pair == PAIR_SWAP) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float t = v[2 * j];
      v[2 * j] = v[2 * j + 1];
      v[2 * j + 1] = t;
    }
  }
}

template <int KIND, int BN, int CTAS, int KS, int KC, int EM>
__global__ void __launch_bounds__(384, 1)
gemm_evt_kernel(const __grid_constant__ GemmParams p) {
  using C = TileCfg<KIND, BN, CTAS, KS, KC>;
  constexpr int STAGES = C::STAGES;
  constexpr int CLUSTER = C::CLUSTER;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

  uint8_t* stage_base = smem;
  uint8_t* epi_base = smem + STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_base + C::EPI_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]   TMA bytes landed (leader CTA's is used)
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]   MMAs reading the stage have finished
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]        accumulator buffer complete
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]    accumulator buffer drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  uint64_t* tail_bar = bars + 2 * STAGES + 6;    // [1]        the CTA's last accumulator is complete
  uint64_t* xfree_bar = bars + 2 * STAGES + 7;   // [1]  KC>1: the other K groups' stages are idle
  uint64_t* xdata_bar = bars + 2 * STAGES + 8;   // [1]  KC>1: their partial accumulators have landed
  uint64_t* opnd_bar = bars + 2 * STAGES + 9;    // [1]  the last tile's staged epilogue operand has landed
  uint64_t* res_bar = bars + 2 * STAGES + 10;    // [12 warps][2]  a warp's residual slice has landed in its staging buffer

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Rank inside the cluster = K group * CTAS + rank inside the MMA pair (cta_group::2 pairs the two
  // CTAs whose cluster ranks differ in the last bit).
  const uint32_t cluster_rank = (CLUSTER > 1) ? ptx::cluster_ctarank() : 0u;
  const uint32_t cta_rank = cluster_rank & static_cast<uint32_t>(CTAS - 1);
  const uint32_t kc = cluster_rank / CTAS;            // this pair's K group, 0 when KC == 1
  const uint32_t pair_base = kc * CTAS;               // cluster rank of this pair's leader
  const int cluster_idx = (CLUSTER > 1) ? static_cast<int>(ptx::cluster_id_x()) : blockIdx.x;
  const int num_clusters = (CLUSTER > 1) ? static_cast<int>(ptx::num_clusters_x()) : gridDim.x;
  const int xchg_warps = (p.diag & 16) ? C::EPI_WARPS : C::EPI_WARPS + 4;   // warps in the exchange
  const int total_items = p.total_items;
  const long long budget = p.wait_budget;

  // The full-matrix epilogue operand of the CTA's last tile is staged in shared memory when one
  // tile of it fits a pipeline stage (and the variant keeps its idle stages free for it).
  const bool tail_opnd = (KC == 1) && (EM & (EF_MAT | EF_ROPE)) && p.tail_opnd != 0 &&
                         p.tail_opnd_boxes * 16384 <= C::STAGE_BYTES && STAGES >= 3;
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&p.tm_a);
    ptx::prefetch_tmap(&p.tm_b);
    if (tail_opnd) ptx::prefetch_tmap(&p.tm_opnd);
    if (!p.direct_store && p.d_dtype == DT_BF16) ptx::prefetch_tmap(&p.tm_d);
  }
  if (warp == 1 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&tfull_bar[b]), 1);
      if (b == 0) {
        ptx::mbar_init(ptx::smem_u32(tail_bar), 1);
        ptx::mbar_init(ptx::smem_u32(xfree_bar), KC > 1 ? KC - 1 : 1);
        ptx::mbar_init(ptx::smem_u32(xdata_bar), KC > 1 ? (KC - 1) * xchg_warps * 32 : 1);
        ptx::mbar_init(ptx::smem_u32(opnd_bar), 1);
        for (int i = 0; i < 2 * (C::EPI_WARPS + 4); ++i) ptx::mbar_init(ptx::smem_u32(&res_bar[i]), 1);
      }
      ptx::mbar_init(ptx::smem_u32(&tempty_bar[b]), C::EPI_WARPS * CTAS);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc<CTAS>(ptx::smem_u32(tmem_slot), C::TMEM_COLS);
    ptx::tmem_relinquish<CTAS>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (CLUSTER > 1) {   // the barrier words were published by fence_mbar_init
    ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  // Programmatic dependent launch.  Everything above touched only shared memory, TMEM and the
  // kernel parameters, so it may run while the previous kernel of the stream is still finishing;
  // nothing below may: every global read and write of this kernel comes after the wait, which
  // returns once the previous grid has completed and its memory is visible.  The early trigger
  // lets the next kernel's CTAs take each SM as soon as this kernel's CTA leaves it.  Both
  // instructions are no-ops for a launch without the attribute.
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = p.l2_hint_a == 1 ? ptx::l2_policy_evict_last()
                                              : (p.l2_hint_a == 2 ? ptx::l2_policy_evict_first() : 0ull);
      const uint64_t pol_b = p.l2_hint_b == 1 ? ptx::l2_policy_evict_last()
                                              : (p.l2_hint_b == 2 ? ptx::l2_policy_evict_first() : 0ull);
      for (int w = cluster_idx; w < total_items && ok; w += num_clusters) {
        const WorkItem wi = decode_item(p, schedule_item(p, w, cluster_idx, num_clusters));
        const TileCoord tc = decode_tile(p, wi.tile);
        const int row0 = (tc.tm * CTAS + static_cast<int>(cta_rank)) * C::BM;
        const int col0 = tc.tn * BN + static_cast<int>(cta_rank) * C::BN_CTA;
        const int la = p.a_batched ? tc.l : 0;
        const int lb = p.b_batched ? tc.l : 0;
        // cluster split-K: this pair takes the kc-th of KC equal parts of the item's K range
        const int kb_lo = (KC > 1) ? wi.kb0 + static_cast<int>(kc) * (wi.kb1 - wi.kb0) / KC : wi.kb0;
        const int kb_hi = (KC > 1) ? wi.kb0 + static_cast<int>(kc + 1) * (wi.kb1 - wi.kb0) / KC : wi.kb1;
        // (Every tile walks K from its first block.  Starting tiles that share an operand panel at
        // different K blocks was tried and is slower: CTAs that ask L2 for the same lines at the
        // same time are served together.)
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, budget)) {
            if (p.status) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_PRODUCER_EMPTY);
            ok = false;
            break;
          }
          const uint32_t my_full = ptx::smem_u32(&full_bar[stage]);
          const uint32_t full_addr = (CTAS == 2) ? ptx::mapa(my_full, pair_base) : my_full;
          if (p.diag & 1) {  // diagnostics: no operand traffic, the stage is "full" at once
            if (cta_rank == 0) ptx::mbar_arrive(my_full);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          if (cta_rank == 0) ptx::mbar_arrive_expect_tx(my_full, C::STAGE_BYTES * CTAS);
          uint8_t* sa = stage_base + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            int ka = kb * C::KBLK + ks * C::KSLAB, a2 = la;
            if (p.a_k_slab > 0) {  // A gathered from column shards: slab index is the third mode
              a2 = ka / p.a_k_slab;
              ka -= a2 * p.a_k_slab;
            }
            if (p.l2_hint_a)
              ptx::tma_load_3d_hint<CTAS>(ptx::smem_u32(sa + ks * C::A_SLAB_BYTES), &p.tm_a, full_addr, ka,
                                          row0, a2, pol_a);
            else
              ptx::tma_load_3d<CTAS>(ptx::smem_u32(sa + ks * C::A_SLAB_BYTES), &p.tm_a, full_addr, ka,
                                     row0, a2);
          }
#pragma unroll
          for (int g = 0; g < C::NGRP; ++g) {
            if (p.l2_hint_b)
              ptx::tma_load_3d_hint<CTAS>(ptx::smem_u32(sb + g * C::GRP_BYTES), &p.tm_b, full_addr,
                                          col0 + g * C::GRP_COLS, kb * C::KBLK, lb, pol_b);
            else
              ptx::tma_load_3d<CTAS>(ptx::smem_u32(sb + g * C::GRP_BYTES), &p.tm_b, full_addr,
                                     col0 + g * C::GRP_COLS, kb * C::KBLK, lb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if constexpr (KC > 1) {
          // One tile per cluster.  The stage that would take the next K block is the first one the
          // MMAs leave: it becomes the buffer the other K groups write their partials into, and they
          // are told as soon as it is idle, a couple of K blocks before the accumulator is complete.
          if (ok && ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, budget)) {
#pragma unroll
            for (int g = 0; g < KC; ++g)
              if (g != static_cast<int>(kc))
                ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(xfree_bar), g * CTAS + cta_rank));
          } else if (ok && p.status) {
            atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_PRODUCER_EMPTY);
          }
          break;
        }
        if (tail_opnd && ok && w + num_clusters >= total_items && wi.split_idx < 0) {
          // Last tile of this CTA: the stage that would take the next K block is the first one the
          // MMAs leave; it receives this CTA's 128 rows of the operand (own barrier, own memory).
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, budget)) {
            if (p.status) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_PRODUCER_EMPTY);
            break;
          }
          const uint32_t ob = ptx::smem_u32(opnd_bar);
          ptx::mbar_arrive_expect_tx(ob, static_cast<uint32_t>(p.tail_opnd_boxes) * 16384u);
          const uint32_t dst = ptx::smem_u32(stage_base + stage * C::STAGE_BYTES);
          const int box_cols = p.tail_opnd == 1 ? 64 : 32;
          const int c0 = p.tail_opnd == 1 ? tc.tn * BN : 0;   // the table is read from its first column
          for (int b = 0; b < p.tail_opnd_boxes; ++b)
            ptx::tma_load_3d<1>(dst + static_cast<uint32_t>(b) * 16384u, &p.tm_opnd, ob, c0 + b * box_cols,
                                row0, tc.l);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc<KIND, BN, CTAS>();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int w = cluster_idx; w < total_items && ok; w += num_clusters, ++it) {
        const WorkItem wi = decode_item(p, schedule_item(p, w, cluster_idx, num_clusters));
        const int buf = it & 1;
        if (!ptx::mbar_wait(ptx::smem_u32(&tempty_bar[buf]), ((it >> 1) & 1) ^ 1u, budget)) {
          if (p.status) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_MMA_TMEM_EMPTY);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        const int kb_lo = (KC > 1) ? wi.kb0 + static_cast<int>(kc) * (wi.kb1 - wi.kb0) / KC : wi.kb0;
        const int kb_hi = (KC > 1) ? wi.kb0 + static_cast<int>(kc + 1) * (wi.kb1 - wi.kb0) / KC : wi.kb1;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, budget)) {
            if (p.status) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_MMA_FULL);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(stage_base + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          const uint64_t adesc = ptx::make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = ptx::make_smem_desc_sw128(sb, C::GRP_BYTES, 1024);
          constexpr int MMAS_PER_SLAB = C::KSLAB / C::UK;  // 4
#pragma unroll
          for (int k = 0; k < KS * MMAS_PER_SLAB; ++k) {
            if (p.diag & 2) break;  // diagnostics: barrier traffic only
            // A: next slab every 4 MMAs, +32 B along K inside the 128-B swizzled row;
            // B: +UK rows of 128 B per MMA
            const int a_off = (k / MMAS_PER_SLAB) * C::A_SLAB_BYTES + (k % MMAS_PER_SLAB) * 32;
            ptx::umma<KIND, CTAS>(d_tmem, adesc + static_cast<uint64_t>(a_off >> 4),
                                  bdesc + static_cast<uint64_t>(k * ((C::UK * 128) >> 4)), idesc,
                                  (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          const uint32_t eb = ptx::smem_u32(&empty_bar[stage]);
          ptx::umma_commit<CTAS>(eb);
          if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(eb, pair_base + 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        const uint32_t tb = ptx::smem_u32(&tfull_bar[buf]);
        ptx::umma_commit<CTAS>(tb);
        if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(tb, pair_base + 1));
        if (w + num_clusters >= total_items || KC > 1) {   // last item: also wake the warps that help with it
          const uint32_t lb = ptx::smem_u32(tail_bar);
          ptx::umma_commit<CTAS>(lb);
          if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(lb, pair_base + 1));
        }
        if constexpr (KC > 1) break;
      }
    }
  }
  __syncwarp();
  {
    // ------------------------------------------------------------------ epilogue
    // Warps 4-11: two warps share each TMEM lane quadrant and take alternate 32-output-column
    // units of the tile, so every scheduler of the SM holds two epilogue warps whose latencies
    // overlap.  Warps 0-3 have finished their own roles by the time the CTA's LAST tile is
    // accumulated, and that tile's epilogue has no main loop left to hide behind: they join it as
    // a third worker per quadrant (a warp may read the TMEM lanes of quadrant warp % 4), staging
    // their stores in the then idle pipeline stages.
    const bool helper = warp < 4;
    const int ew = helper ? warp : warp - 4;
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = helper ? 2 : ew >> 2;  // which worker of the quadrant
    const EpiParams& e = p.epi;
    uint8_t* stg = helper ? stage_base + warp * (C::EPI_BUFS * C::EPI_BUF_BYTES)
                          : epi_base + ew * (C::EPI_BUFS * C::EPI_BUF_BYTES);
    int sidx = 0;
    uint32_t res_phase = 0;                 // parity bits of this warp's two residual-slice barriers
    bool res_failed = false;
    int kb_seen = 0;                        // K blocks this CTA's pipeline has carried so far
    const uint8_t* staged = nullptr;        // the last tile's operand tile in shared memory, if staged
    const bool compact = (EM & EF_GLU) ? e.compact != 0 : false;
    const int n_out = compact ? (p.N >> 1) : p.N;
    const int slices_per_unit = compact ? 2 : 1;   // 32 output columns = 1 or 2 accumulator slices
    const uint32_t tempty_leader =
        (CTAS == 2) ? ptx::mapa(ptx::smem_u32(&tempty_bar[0]), pair_base) : ptx::smem_u32(&tempty_bar[0]);
    const int pre_which = preload_choice<EM>(e);
    int it = 0;
    for (int w = cluster_idx; w < total_items; w += num_clusters, ++it) {
      if (KC > 1 && it > 0) break;   // cluster split-K: one tile per cluster
      const WorkItem wi = decode_item(p, schedule_item(p, w, cluster_idx, num_clusters));
      // the CTA's last item, if it is a whole tile, is shared three ways per quadrant
      const bool shared3 = (w + num_clusters >= total_items || KC > 1) && wi.split_idx < 0 && !(p.diag & 16);
      kb_seen += wi.kb1 - wi.kb0;
      const bool use_staged = tail_opnd && (w + num_clusters >= total_items) && wi.split_idx < 0;
      if (KC > 1 && helper) {   // off the stage that receives the other groups' partials
        const int nkb_item = wi.kb1 - wi.kb0;
        const int mine = (nkb_item * (static_cast<int>(kc) + 1) / KC - nkb_item * static_cast<int>(kc) / KC) % STAGES;
        stg = stage_base + ((mine + 1) % STAGES) * C::STAGE_BYTES + warp * (C::EPI_BUFS * C::EPI_BUF_BYTES);
      }
      if (use_staged) {
        // the producer put the operand in the stage after the last K block's; the helpers' store
        // staging moves to the stage after that one
        const int sx = kb_seen % STAGES;
        staged = stage_base + sx * C::STAGE_BYTES;
        if (helper)
          stg = stage_base + ((sx + 1) % STAGES) * C::STAGE_BYTES + warp * (C::EPI_BUFS * C::EPI_BUF_BYTES);
      }
      const TileCoord tc = decode_tile(p, wi.tile);
      const int buf = it & 1;
      const int m0 = (tc.tm * CTAS + static_cast<int>(cta_rank)) * C::BM;
      const int n0 = tc.tn * BN;
      const int l = tc.l;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      float rs = 1.0f;
      if (e.row_scale.enabled && row_ok && (!helper || shared3))
        rs = load_vec_elem(e.row_scale, static_cast<long long>(l) * e.row_scale.batch_stride + row);
      // while the tile's main loop runs: bring this row's residual / cos_sin lines into L2
      if ((EM & (EF_MAT | EF_ROPE)) && !helper && row_ok && pre_which != PRE_NONE && p.d_dtype != DT_S32)
        prefetch_tile_operands<EM>(e, p.N, l, row, n0, min(BN, p.N - n0), half, 2);

      // Helpers wait on a barrier of their own that completes once, with the CTA's last
      // accumulator: the two-phase barriers of the accumulator buffers name a phase by one parity
      // bit, which a warp that has not followed them phase by phase cannot wait on safely.
      if (helper) {
        if (!shared3) continue;
        if (!ptx::mbar_wait(ptx::smem_u32(tail_bar), 0u, budget)) {
          if (p.status && lane == 0) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_EPI_TMEM_FULL);
          break;
        }
      } else if (!ptx::mbar_wait(ptx::smem_u32(&tfull_bar[buf]), (it >> 1) & 1, budget)) {
        if (p.status && lane == 0) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_EPI_TMEM_FULL);
        break;
      }
      ptx::tc_fence_after();
      if (use_staged && !ptx::mbar_wait(ptx::smem_u32(opnd_bar), 0u, budget)) {
        if (p.status && lane == 0) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_EPI_OPERAND);
        break;
      }

      const uint32_t t_row = tmem_base + static_cast<uint32_t>(buf * BN) +
                             (static_cast<uint32_t>(q * 32) << 16);
      const int ncols_tile = min(BN, p.N - n0);           // valid accumulator columns
      const bool warp_rows_ok = (m0 + q * 32) < p.M;      // any row of this warp inside M
      const int nsub = (ncols_tile + 31) / 32;            // 32-column accumulator slices
      const int nunits = (nsub + slices_per_unit - 1) / slices_per_unit;
      bool released = false;
      const bool last_item = (w + num_clusters >= total_items) || KC > 1;
      auto release_tmem = [&]() {   // this warp has read its last slice of the accumulator buffer
        released = true;
        // nobody waits for the buffer of the CTA's last item (helpers only ever see that one): its
        // epilogue is not hidden by anything, and the cluster-scope release costs it ~0.5 us
        if (helper || last_item) return;
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader + static_cast<uint32_t>(buf * 8));
      };

      // Split tile.  Every slice publishes its raw accumulator rows, then the S slices share the
      // finishing work: slice i sums, in slice order, the 32-output-column units u = i (mod S) of
      // all S partials and runs the epilogue on them.  A slice is the first item of its CTA and
      // depends on nothing but the other slices' first items, and all CTAs of the grid are or
      // become resident, so the wait below cannot deadlock; it is bounded all the same.
      const float* part_base = nullptr;   // non-null: accumulators come from the partials, not TMEM
      int* split_ctr = nullptr;           // [0] warps that have published, [1] warps that are done
      int u_first = half, u_step = shared3 ? 3 : 2;
      if (wi.split_idx >= 0) {
        const size_t slab = static_cast<size_t>(C::BM) * BN;   // words per (slice, CTA)
        // slab layout [32-column slice][16-byte chunk][row]: the 32 lanes of a store are contiguous
        uint4* mine = reinterpret_cast<uint4*>(
                          p.split_partials +
                          ((static_cast<size_t>(wi.split_idx) * p.split_s + wi.slice) * CTAS + cta_rank) * slab) +
                      (q * 32 + lane);
        for (int u = half; u < nunits; u += 2) {
          for (int h = 0; h < slices_per_unit; ++h) {
            const int s = u * slices_per_unit + h;
            if (s >= nsub) break;
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(s * 32), r);
            ptx::tmem_ld_wait();
            uint4* dst = mine + static_cast<size_t>(s) * 8 * C::BM;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[j * C::BM] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          }
        }
        release_tmem();
        __threadfence();
        __syncwarp();
        split_ctr = p.split_counters + (wi.split_idx * CTAS + static_cast<int>(cta_rank)) * 8;
        if (lane == 0) atomicAdd(split_ctr, 1);
        u_first = wi.slice + p.split_s * half;
        u_step = 2 * p.split_s;
        if (u_first < nunits) {
          int seen_all = 1;
          if (lane == 0) {
            const int target = C::EPI_WARPS * p.split_s;
            const long long t0 = clock64();
            while (ptx::ld_acquire_gpu(split_ctr) < target) {
              if (clock64() - t0 > budget) { seen_all = 0; break; }
              __nanosleep(64);
            }
          }
          seen_all = __shfl_sync(0xffffffffu, seen_all, 0);
          __threadfence();
          if (!seen_all) {
            if (p.status && lane == 0) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_SPLIT_PARTIALS);
            u_first = nunits;   // nothing to finish; fall through to the bookkeeping
          }
        }
        part_base = p.split_partials + (static_cast<size_t>(wi.split_idx) * p.split_s * CTAS + cta_rank) * slab +
                    static_cast<size_t>(q * 32 + lane) * 4;
      }

      // Cluster split-K.  Every CTA of the cluster holds, for its 128 rows, the partial accumulator of
      // its pair's K range over all BN columns.  K group g finishes columns [g*BN/KC, (g+1)*BN/KC):
      // each CTA sends the other groups' columns of its partial to the CTA with the same rows in that
      // group (st.shared::cluster into its idle pipeline stages) and receives KC-1 partials of its own
      // columns, which the unit loop below adds, in group order, to what it reads from TMEM.
      int u_end = nunits;
      const uint4* xrecv = nullptr;
      if constexpr (KC > 1) {
        constexpr int SPG = C::XCHG_SLICES;
        const uint32_t xfree = ptx::smem_u32(xfree_bar), xdata = ptx::smem_u32(xdata_bar);
        const int workers = shared3 ? 3 : 2;
        const int nkb_item = wi.kb1 - wi.kb0;
        // receive stage of K group g: the ring slot after its last K block (its producer said so)
        auto recv_stage = [&](int g) { return (nkb_item * (g + 1) / KC - nkb_item * g / KC) % STAGES; };
        bool ok = true;
        // every other group's receive stage is idle (signalled by its producer warp)
        if (!ptx::mbar_wait_cluster(xfree, 0u, budget)) ok = false;
        if (ok) {
          for (int idx = half; idx < (KC - 1) * SPG; idx += workers) {
            const int gslot = idx / SPG, sl = idx - gslot * SPG;
            const int g = gslot < static_cast<int>(kc) ? gslot : gslot + 1;      // destination K group
            const int slot = static_cast<int>(kc) < g ? static_cast<int>(kc) : static_cast<int>(kc) - 1;
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(g * (BN / KC) + sl * 32), r);
            ptx::tmem_ld_wait();
            // receiver layout [sender slot][slice][16-byte chunk][row]: a warp's store is 512 contiguous bytes
            const uint32_t xbuf = ptx::smem_u32(stage_base + recv_stage(g) * C::STAGE_BYTES);
            const uint32_t dst = ptx::mapa(xbuf, g * CTAS + cta_rank) +
                                 static_cast<uint32_t>((((slot * SPG + sl) * 8) * C::BM + q * 32 + lane) * 16);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              ptx::st_shared_cluster_v4(dst + static_cast<uint32_t>(j * C::BM * 16),
                                        make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
          }
        }
        // every thread releases its own stores to every other group, then waits for theirs
#pragma unroll
        for (int g = 0; g < KC; ++g)
          if (g != static_cast<int>(kc)) ptx::mbar_arrive_cluster(ptx::mapa(xdata, g * CTAS + cta_rank));
        if (ok && !ptx::mbar_wait_cluster(xdata, 0u, budget)) ok = false;
        if (!ok) {
          if (p.status && lane == 0) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_CLUSTER_EXCHANGE);
          break;
        }
        const int upg = SPG / slices_per_unit;                  // output units per K group
        u_first = static_cast<int>(kc) * upg + half;
        u_end = min(nunits, (static_cast<int>(kc) + 1) * upg);
        xrecv = reinterpret_cast<const uint4*>(stage_base + recv_stage(static_cast<int>(kc)) * C::STAGE_BYTES) +
                (q * 32 + lane);
      }

      // One 32-register group per thread serves two purposes.  Where the epilogue reads a residual /
      // cos_sin operand from global memory it holds that operand's words, requested before the
      // accumulator slice is read.  Otherwise (no such operand, or the operand staged in shared
      // memory) it receives the NEXT accumulator slice of this warp while the current one is being
      // processed, so the TMEM read latency is paid once per tile instead of once per slice.
      uint4 pre[8];
      // residual slices by TMA into the buffer the result will be stored from (bf16 TMA-store path only)
      const bool res_by_tma = (EM & EF_MAT) && p.res_tma != 0 && pre_which == PRE_RESIDUAL && !use_staged && !compact &&
                              !p.direct_store && p.d_dtype == DT_BF16 && warp_rows_ok && !(p.diag & (4 | 8));
      // the auxiliary output through a staging buffer and a TMA store (same conditions as the D store)
      const bool aux_by_tma = (EM & EF_MAT) && p.aux_tma != 0 && !compact && !p.direct_store && p.d_dtype == DT_BF16 &&
                              warp_rows_ok && !(p.diag & (4 | 8));
      const bool acc_prefetch = part_base == nullptr && (pre_which == PRE_NONE || use_staged) && !(p.diag & 32);
      bool prefetched = false;
      for (int u = u_first; u < u_end; u += u_step) {
        uint32_t pk[16];
        int out_col0 = 0;
        bool stored_direct = false;
#pragma unroll 1
        for (int h = 0; h < slices_per_unit; ++h) {
          const int s = u * slices_per_unit + h;
          if (s >= nsub) break;   // odd slice count at the N edge of a compact tile
          float v[32];
          uint32_t r[32];
          const int tcol0 = s * 32;
          // the residual / cos_sin loads of this slice go out before the accumulator is read
          int pre_mode = 0;
          if (res_by_tma) {
            // the buffer this slice's store will use: free once the store of two slices ago has read it
            if (lane == 0) {
              ptx::tma_store_wait_read<C::EPI_BUFS - 1>();
              const uint32_t rb = ptx::smem_u32(&res_bar[warp * 2 + sidx]);
              ptx::mbar_arrive_expect_tx(rb, C::EPI_BUF_BYTES);
              ptx::tma_load_3d<1>(ptx::smem_u32(stg + sidx * C::EPI_BUF_BYTES), &p.tm_res, rb, n0 + tcol0,
                                  m0 + q * 32, l);
            }
          } else if (!acc_prefetch && !use_staged && row_ok && !(p.diag & 4) && p.d_dtype != DT_S32) {
            if ((EM & EF_MAT) && pre_which == PRE_RESIDUAL)
              pre_mode = mat_row32_issue(e.residual, l, row, n0 + tcol0, p.N, pre);
            else if ((EM & EF_ROPE) && pre_which == PRE_COS_SIN)
              pre_mode = mat_row32_issue(e.cos_sin, l, row, cos_sin_col(e, n0 + tcol0), cos_sin_width(e, p.N), pre);
          }
          if (part_base == nullptr) {
            // this warp's next slice of the tile, if any
            const bool more_in_unit = (h + 1 < slices_per_unit) && (s + 1 < nsub);
            const bool has_next = more_in_unit || (u + u_step < u_end);
            const int next_s = more_in_unit ? s + 1 : (u + u_step) * slices_per_unit;
            if (prefetched) {
              ptx::tmem_ld_wait_for(pre);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                r[4 * j] = pre[j].x; r[4 * j + 1] = pre[j].y; r[4 * j + 2] = pre[j].z; r[4 * j + 3] = pre[j].w;
              }
              prefetched = false;
            } else if (p.diag & 64) {   // diagnostics: no accumulator read
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0u;
            } else {
              ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(tcol0), r);
              ptx::tmem_ld_wait();
            }
            if (acc_prefetch && has_next && !(p.diag & 64)) {
              ptx::tmem_ld_32x32_async(t_row + static_cast<uint32_t>(next_s * 32), pre);
              prefetched = true;
            }
            if (!has_next) release_tmem();
            if constexpr (KC > 1) {
              // add the other K groups' partials of this slice, in group order
              const int sl = s - static_cast<int>(kc) * C::XCHG_SLICES;
#pragma unroll
              for (int slot = 0; slot < KC - 1; ++slot) {
                const uint4* src = xrecv + static_cast<size_t>((slot * C::XCHG_SLICES + sl) * 8) * C::BM;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const uint4 x = src[j * C::BM];
                  const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                  for (int t = 0; t < 4; ++t) {
                    if constexpr (KIND == 0)
                      r[4 * j + t] = __float_as_uint(__uint_as_float(r[4 * j + t]) + __uint_as_float(xs[t]));
                    else
                      r[4 * j + t] = static_cast<uint32_t>(static_cast<int>(r[4 * j + t]) + static_cast<int>(xs[t]));
                  }
                }
              }
            }
          } else {
            // sum the slices in slice order (the same order whichever slice arrived last); L2 loads:
            // the partials were written by other SMs
            const size_t slice_stride = static_cast<size_t>(CTAS) * C::BM * BN;
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
            const uint4* src0 = reinterpret_cast<const uint4*>(part_base) + static_cast<size_t>(s) * 8 * C::BM;
            const size_t slice_stride4 = slice_stride / 4;
            auto add4 = [&](int j, const uint4& x) {
              const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                if constexpr (KIND == 0)
                  r[4 * j + t] = __float_as_uint(__uint_as_float(r[4 * j + t]) + __uint_as_float(xs[t]));
                else
                  r[4 * j + t] = static_cast<uint32_t>(static_cast<int>(r[4 * j + t]) + static_cast<int>(xs[t]));
              }
            };
            int sl = 0;
            for (; sl + 2 <= p.split_s; sl += 2) {   // two slices (16 loads) in flight per lane
              uint4 x0[8], x1[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                x0[j] = __ldcg(src0 + sl * slice_stride4 + j * C::BM);
                x1[j] = __ldcg(src0 + (sl + 1) * slice_stride4 + j * C::BM);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) add4(j, x0[j]);
#pragma unroll
              for (int j = 0; j < 8; ++j) add4(j, x1[j]);
            }
            if (sl < p.split_s) {
#pragma unroll
              for (int j = 0; j < 8; ++j) add4(j, __ldcg(src0 + sl * slice_stride4 + j * C::BM));
            }
          }
          if (p.diag & 4) { stored_direct = true; continue; }  // diagnostics: TMEM drain only
          if ((EM & EF_MISC) && p.d_dtype == DT_S32) {
            // raw int32 accumulator, no epilogue steps (checked on the host)
            if (row_ok) {
              int* dp = reinterpret_cast<int*>(p.D) + static_cast<long long>(l) * p.batch_d +
                        static_cast<long long>(row) * p.ldd + n0 + tcol0;
              const int nv = p.N - (n0 + tcol0);
              if (nv >= 32 && (reinterpret_cast<uintptr_t>(dp) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  reinterpret_cast<uint4*>(dp)[j] =
                      make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i < nv) dp[i] = static_cast<int>(r[i]);
              }
            }
            stored_direct = true;
            continue;
          }
          if (res_by_tma) {
            const uint32_t rb = ptx::smem_u32(&res_bar[warp * 2 + sidx]);
            if (!ptx::mbar_wait(rb, (res_phase >> sidx) & 1u, budget)) {
              if (p.status && lane == 0) atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_EPI_OPERAND);
              res_failed = true;
            }
            res_phase ^= 1u << sidx;
            const uint8_t* sb = stg + sidx * C::EPI_BUF_BYTES + lane * 64;
            const int sw = (lane >> 1) & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) pre[j] = *reinterpret_cast<const uint4*>(sb + ((j ^ sw) << 4));
            pre_mode = 1;
          }
          if (aux_by_tma && !res_by_tma) {   // the buffer the auxiliary block leaves from must be free
            if (lane == 0) ptx::tma_store_wait_read<C::EPI_BUFS - 1>();
            __syncwarp();
          }
          epilogue_chunk<KIND, EM>(e, p.N, r, v, row, row_ok, l, n0 + tcol0, rs, pre_which, pre_mode, pre,
                               use_staged ? staged : nullptr, q * 32 + lane,
                               pre_which == PRE_RESIDUAL ? tcol0 : cos_sin_col(e, n0 + tcol0),
                               aux_by_tma ? stg + sidx * C::EPI_BUF_BYTES + lane * 64 : nullptr, (lane >> 1) & 3);
          if (aux_by_tma) {
            // (with the residual fetched by TMA this is the buffer it arrived in: every lane has read
            // its row and overwritten it with the auxiliary values)
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_3d(&p.tm_aux, ptx::smem_u32(stg + sidx * C::EPI_BUF_BYTES), n0 + tcol0, m0 + q * 32, l);
              ptx::tma_store_commit();
            }
            sidx = (sidx + 1 == C::EPI_BUFS) ? 0 : sidx + 1;
          }
          if ((EM & EF_MISC) && e.row_sumsq != nullptr) {
            // side output for a following RMSNorm: this row's sum of squares over these 32 columns
            const int nv = p.N - (n0 + tcol0);
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) ss += (i < nv) ? v[i] * v[i] : 0.0f;
            if (row_ok) {
              const long long units = (p.N + 31) >> 5;
              e.row_sumsq[(static_cast<long long>(l) * units + ((n0 + tcol0) >> 5)) * p.M + row] = ss;
            }
          }
          if ((EM & EF_MISC) && p.d_dtype == DT_F32) {
            if (row_ok) {
              float* dp = reinterpret_cast<float*>(p.D) + static_cast<long long>(l) * p.batch_d +
                          static_cast<long long>(row) * p.ldd + n0 + tcol0;
              const int nv = p.N - (n0 + tcol0);
              if (nv >= 32 && (reinterpret_cast<uintptr_t>(dp) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  reinterpret_cast<float4*>(dp)[j] =
                      make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i < nv) dp[i] = v[i];
              }
            }
            stored_direct = true;
            continue;
          }
          if (!compact) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
            out_col0 = n0 + tcol0;
          } else if (h == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) pk[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
            out_col0 = (n0 + tcol0) >> 1;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) pk[8 + i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
          }
        }
        if (stored_direct || (p.diag & 8)) continue;
        // bf16 output: 32 output columns (64 bytes per row) per store
        if ((EM & EF_MISC) && p.direct_store) {
          if (row_ok) {
            __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) +
                                static_cast<long long>(l) * p.batch_d +
                                static_cast<long long>(row) * p.ldd + out_col0;
            store_bf16_row(dp, pk, n_out - out_col0, 32);
            for (int c = 0; c < p.num_d_peer; ++c) {
              __nv_bfloat16* pp = reinterpret_cast<__nv_bfloat16*>(p.D_peer[c]) +
                                  static_cast<long long>(l) * p.batch_d +
                                  static_cast<long long>(row) * p.ldd + out_col0;
              store_bf16_row(pp, pk, n_out - out_col0, 32);
            }
          }
        } else if (warp_rows_ok) {
          if (lane == 0) ptx::tma_store_wait_read<C::EPI_BUFS - 1>();  // oldest staging buffer is free
          __syncwarp();
          uint8_t* sbuf = stg + sidx * C::EPI_BUF_BYTES;
          const int sw = (lane >> 1) & 3;  // 64-B swizzle: 16-B chunk index ^= address bits [7,9)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(sbuf + lane * 64 + ((j ^ sw) << 4)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            ptx::tma_store_3d(&p.tm_d, ptx::smem_u32(sbuf), out_col0, m0 + q * 32, l);
            // the same tile into every peer's gathered buffer: the all-gather rides on the epilogue
            for (int c = 0; c < p.num_d_peer; ++c)
              ptx::tma_store_3d(&p.tm_d_peer[c], ptx::smem_u32(sbuf), out_col0, m0 + q * 32, l);
            ptx::tma_store_commit();
          }
          sidx = (sidx + 1 == C::EPI_BUFS) ? 0 : sidx + 1;
        }
      }
      if (!released) release_tmem();   // this warp had no unit in the tile (narrow tile at the N edge)
      if (split_ctr != nullptr) {
        // The last warp of the last slice to get here knows every wait above has ended: it leaves
        // both counters at zero for the next launch.
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          if (atomicAdd(split_ctr + 1, 1) == C::EPI_WARPS * p.split_s - 1) {
            split_ctr[0] = 0;
            split_ctr[1] = 0;
          }
        }
      }
    }
    // Before the CTA may exit its staging buffers must have been read by the bulk stores; the
    // writes themselves complete with the grid.  Stores into another GPU's memory are waited for
    // in full: the host-side barrier that follows the kernel tells the peers their data has landed.
    if (lane == 0) {
      if (p.num_d_peer > 0) ptx::tma_store_wait_all<0>();
      else ptx::tma_store_wait_read<0>();
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  // No CTA leaves while a peer may still write its barriers or stages, or read the pair's TMEM.
  // Only execution is ordered here: every remote write was waited for through an mbarrier before the
  // epilogue used it, and a releasing arrival would also wait for this CTA's outstanding output
  // stores (0.65 us at the end of every launch).
  if constexpr (CLUSTER > 1) {
    ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CTAS>(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace xf
