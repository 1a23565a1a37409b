// The tcgen05 GEMM of the path: one persistent, warp-specialised kernel that
// serves the dense baseline, the rank-7 product walk (all products per tile, or
// one product per work unit) and the chained gate_up form whose extra warps turn
// finished Z tiles into the consumer's A planes.
//
// Per CTA:  warp 0      TMA producer (one lane)
//           warp 1      TMEM allocation + tcgen05.mma issue (one lane, pair leader only)
//           warps 2-5   epilogue: TMEM -> registers -> bf16 -> swizzled smem -> TMA store / reduce-add
//           warps 6-13  (chain only) SwiGLU + A planes of the tile finished before
//
// Data flow per accumulator step t of a work unit:
//   A plane tile (128 x 64 bf16 per CTA) and B plane tile (256 / group x 64) arrive by TMA
//   with the 128-byte swizzle, tcgen05.mma accumulates 128 x 256 fp32 per CTA in TMEM stage
//   t % 2 (a step that does not clear adds to the sum left by step t - 2: the chain
//   trick of lcgemm/scheme.py:18-40), the epilogue publishes the stage to the C blocks the
//   plan names (lcgemm/kernels/sm100.py:690-727).
//
// Every wait is bounded (lcg_ptx.cuh: mbar_wait); a wait that runs out flags the CTA and
// the status word and the kernel finishes without blocking again.
#include <cuda_bf16.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "lcg_common.h"
#include "lcg_ptx.cuh"

namespace lcg {

constexpr int kBM = 128;        // accumulator rows per CTA = TMEM lanes
constexpr int kBN = 256;        // accumulator columns per stage
constexpr int kBK = 64;         // K per pipeline stage (one 128-byte swizzle row)
constexpr int kUmmaK = 16;      // K per tcgen05.mma, bf16
constexpr int kEpiCols = 64;    // columns per staged epilogue sub-tile
constexpr int kEpiBytes = kBM * kEpiCols * 2;
constexpr int kEpiBufs = 2;
// Rows per TMA store / reduce-add of the epilogue.  A staged 128 x 64 sub-tile leaves as four
// 32-row operations rather than one: the TMA unit serves the operand loads from the same queue,
// and a 16 KiB store in front of a load adds its whole transfer time to the stage-recycle loop
// (measured on gate_up at 4096 tokens: 128 rows 889 us, 64 rows 886, 32 rows 877, 16 rows 890,
// 8 rows 913).
constexpr int kEpiBoxRows = 32;
constexpr uint32_t kTmemCols = 512;
constexpr int kPlaneThreads = 256;
constexpr int kThreadsPlain = 192;
constexpr int kThreadsChain = 512;

// Which warp plays which part.  A warp issues from scheduler (warp % 4) of the SM, and an
// epilogue warp reads the TMEM lane quarter (warp % 4), so one epilogue warp sits on every
// scheduler whatever the layout.  The two single-thread warps that drive the operand ring (TMA
// producer, MMA issuer) are on its critical loop: every cycle one of their instructions waits
// for an issue slot is a cycle added to the stage-recycle round trip.  In the chained kernel the
// eight plane warps are busy SIMT code, so they stay off the scheduler those two live on:
//   plain   (6 warps):  0 producer, 1 MMA, 2-5 epilogue
//   chained (16 warps): 0 producer, 4 MMA (both scheduler 0), 1 2 3 8 epilogue,
//                       5 6 7 9 10 11 13 14 plane warps (schedulers 1-3), 12 15 idle
//   fused-A (16 warps): the chained layout with the plane warps' seats taken by the eight warps that
//                       form the A operand tiles in shared memory
template <bool kChain>
struct Roles {
  static constexpr int kProducer = 0;
  static constexpr int kMma = kChain ? 4 : 1;
  static constexpr int kEpiIssuer = kChain ? 1 : 2;
  __device__ static bool is_epilogue(int warp) {
    return kChain ? (warp == 1 || warp == 2 || warp == 3 || warp == 8) : (warp >= 2 && warp < 6);
  }
  // index 0..7 of a plane warp, or -1
  __device__ static int plane_index(int warp) {
    if (!kChain || (warp & 3) == 0 || warp < 5 || warp > 14) return -1;
    return warp < 8 ? warp - 5 : (warp < 12 ? warp - 6 : warp - 7);
  }
};

// Codes left in the status word by a wait that ran out.
constexpr int kCodeProducer = 101, kCodeMmaAcc = 102, kCodeMmaFull = 103, kCodeEpilogue = 104,
              kCodePlane = 105, kCodeAhead = 107;

template <int kCtaGroup>
struct Tile {
  static constexpr int kBRows = kBN / kCtaGroup;        // B rows each CTA loads
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kCtaGroup == 1 ? 4 : 6;
  static constexpr int kTileM = kBM * kCtaGroup;        // rows per work-unit tile
  static constexpr int kSmemData = kStages * kStageBytes + kEpiBufs * kEpiBytes;
  static constexpr int kSmemBytes = kSmemData + 256 /*barriers*/ + 1024 /*alignment slack*/;
};

struct CMaps {
  CUtensorMap m[4];
};

struct ChainParams {
  const __nv_bfloat16* z;     // the GEMM's own output, re-read L2-hot
  int64_t ldz;
  __nv_bfloat16* planes;      // (plane_rank * m2, inter / 2)
  int64_t ld_planes;
  int32_t m2;                 // rows per block row
  int32_t inter;              // I: S columns; gate block = z[:, :I], up block = z[:, I:]
  int32_t plane_rank;
  int32_t iters_max;          // most work units any CTA group walks
  TermTable plane_terms;
  uint4* preclear;            // consumer output to zero (or to fill from `preload`), or null
  int64_t preclear_vecs;
  const uint4* preload;       // what the consumer output starts from instead of zero, or null
};

// Tensor-parallel push: where the rows of this rank's finished C tiles go.  Row g of the (M, N)
// partial belongs to rank g / rows_per_owner; it is copied to slot[owner], an (rows_per_owner, N)
// row-major region of the owner's memory reserved for this rank (a peer-mapped address, or a
// local one for the rank's own rows), with plain 16-byte stores over NVLink.
constexpr int kMaxWorld = 8;
struct PushParams {
  const __nv_bfloat16* c;
  int64_t ldc;
  __nv_bfloat16* slot[kMaxWorld];
  int32_t world;              // 0: no push
  int32_t rows_per_owner;
  int32_t m, n, m2, n2;
};

// Fused A-side producer: the GEMM reads the activation matrix itself and forms each product's
// A operand tile (the signed sum of one or two of the four blocks of A) on its way into shared
// memory, so no A planes exist in global memory.  Product r reads blocks blk[r][t] = i * 2 + k
// with sign neg[r][t]; a product with a single +1 term is loaded by TMA straight into the operand
// stage (simt[r] = 0), the others go through the eight producer warps' registers.
struct FuseParams {
  const __nv_bfloat16* a;     // (m, K) row-major, leading dimension lda
  int64_t lda;
  int32_t m, m2, k2;
  int8_t nterm[kMaxRank];
  int8_t simt[kMaxRank];
  int8_t blk[kMaxRank][2];
  int8_t neg[kMaxRank][2];
  // Product-ahead form: the two-term products' planes are written to `scratch` (plane slot[r] at
  // rows slot[r] * m2, leading dimension k2) by the plane warps of all CTAs, one product ahead of
  // the MMAs; counters[r] counts the finished chunks of product r's plane (`chunks` when complete).
  __nv_bfloat16* scratch;
  uint32_t* counters;
  int32_t chunks;
  int32_t chunk_rows;
  int8_t slot[kMaxRank];      // -1: single +1 term, read from `a` itself
  int8_t order[kMaxRank];     // products with a plane slot, in the order the steps first need them
  int32_t nslots;
};

struct GemmParams {
  StepDesc steps[kMaxRank];        // whole-tile walk: chain plan, store-first scatter (or the dense step)
  StepDesc steps_split[kMaxRank];  // one product alone, reduce-add only
  int32_t steps_per_unit;     // steps of a whole-tile unit: 7, or 1 (dense)
  // Unit list: [0, main_tiles) whole tiles; then single-product units over the tail_tiles tiles
  // that follow (product-major: q = product * tail_tiles + n), the first full_units of them over
  // the whole K, the remaining split_units each cut into ksplit K ranges (part-major).
  // All-ranks: tail_tiles = 0.  Rank split: main_tiles = 0, tail_tiles = all tiles (and C arrives
  // zeroed by the caller; `zero_tail` = 0).  Hybrid: both parts, tail zeroed by k_zero_tail_tiles.
  int32_t main_tiles;
  int32_t tail_tiles;
  int32_t full_units;
  int32_t split_units;
  int32_t ksplit;
  int32_t zero_tail;
  int32_t tiles_m, tiles_n, group_m;
  int32_t tm_base;            // first tile row of this launch (a slab of tile rows; 0 = from the top)
  int32_t tm_rot;             // the walk starts this many tile rows down and wraps (tensor-parallel push)
  int32_t max_groups;         // cap on CTA groups (0 = all SMs); leaves SMs to a concurrent kernel
  int32_t num_units;
  int32_t k_blocks;
  int32_t a_plane_rows, b_plane_rows;
  int32_t* status;
  ChainParams chain;
  PushParams push;
  FuseParams fuse;
};

// Work unit -> (first step, tile row, tile column).  Tiles are walked in bands of
// group_m tile rows, tile row fastest inside a band, so the tiles in flight at any
// time span a near-square patch and share operand panels in L2
// (lcgemm/kernels/sm100.py:78-96,754-772).
struct UnitCoord {
  int step0, nsteps;   // steps [step0, step0 + nsteps) of the table `split` selects
  int split;           // 1: steps_split (single product, reduce-add), 0: steps
  int tile;            // linear tile index
  int tail;            // index among the tail tiles, or -1
  int kb0, kb1;        // K blocks [kb0, kb1) of every step of the unit
  int tm, tn;
};
__device__ __forceinline__ void tile_coord(const GemmParams& p, int t, int& tm, int& tn) {
  const int band_sz = p.group_m * p.tiles_n;
  const int band = t / band_sz;
  const int rem = t - band * band_sz;
  const int gm = min(p.group_m, p.tiles_m - band * p.group_m);
  tm = band * p.group_m + rem % gm + p.tm_rot;
  tm = p.tm_base + (tm >= p.tiles_m ? tm - p.tiles_m : tm);
  tn = rem / gm;
}
__device__ __forceinline__ UnitCoord decode_unit(const GemmParams& p, int u) {
  UnitCoord c;
  c.kb0 = 0;
  c.kb1 = p.k_blocks;
  if (u < p.main_tiles) {
    c.step0 = 0;
    c.nsteps = p.steps_per_unit;
    c.split = 0;
    c.tile = u;
    c.tail = -1;
  } else {
    int q = u - p.main_tiles;
    if (q >= p.full_units) {          // a K range of one of the last split_units product units
      const int w = q - p.full_units;
      const int part = w / p.split_units;
      q = p.full_units + (w - part * p.split_units);
      c.kb0 = (p.k_blocks * part) / p.ksplit;
      c.kb1 = (p.k_blocks * (part + 1)) / p.ksplit;
    }
    c.step0 = q / p.tail_tiles;
    c.tail = q - c.step0 * p.tail_tiles;
    c.tile = p.main_tiles + c.tail;
    c.nsteps = 1;
    c.split = 1;
  }
  tile_coord(p, c.tile, c.tm, c.tn);
  return c;
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    f[2 * t] = __uint_as_float(w[t] << 16);
    f[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
  }
}

// silu(g) = g / (1 + e^-g) with the fast exponential and reciprocal (2 ulp each); large |g| is safe:
// e^-g -> inf gives -0, e^-g -> 0 gives g.
__device__ __forceinline__ float silu_dev(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// SwiGLU and the consumer's A planes for 32 rows of one tile column: rows [row0, row0 + 32) of
// each block row of Z, S columns [tn * 256, tn * 256 + 256) of the gate and the up block, read
// L2-hot; plane columns [tn * 128, +128).  256 threads: 16 slots across (chunk pair, 8-column
// vector), 16 rows per pass, two passes (16 x 16-byte loads per thread) in flight at a time.
template <unsigned long long kCode>   // packed coefficient table known at compile time, or 0
__device__ __forceinline__ void plane_rows32(const ChainParams& ch, int tn, int row0, int ptid) {
  const int slot = ptid & 15;
  const int pair = slot >> 3;
  const int vc = slot & 7;
  const int rsub = ptid >> 4;
  const int scol = tn * kBN + pair * 128 + vc * 8;     // S column of chunk h = 0
  const int pcol = tn * (kBN / 2) + pair * 64 + vc * 8;
  if (scol + 64 >= ch.inter) return;
  uint4 q[2][2][2][2];
  int rho[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    rho[t] = row0 + rsub + t * 16;
    if (rho[t] < ch.m2) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
            q[t][i][j][hh] = __ldcg(reinterpret_cast<const uint4*>(
                ch.z + (static_cast<int64_t>(i) * ch.m2 + rho[t]) * ch.ldz +
                static_cast<int64_t>(j) * ch.inter + scol + hh * 64));
    }
  }
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    if (rho[t] >= ch.m2) continue;
    float sv[4][8];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float g[8], uu[8];
        unpack_bf16x8(q[t][i][0][hh], g);
        unpack_bf16x8(q[t][i][1][hh], uu);
#pragma unroll
        for (int e = 0; e < 8; ++e) sv[i * 2 + hh][e] = __fmul_rn(silu_dev(g[e]), uu[e]);   // never fused into the sums
      }
    auto store_plane = [&](int r, const float (&o)[8]) {
      uint4 outv;
      outv.x = pack_bf16x2(o[0], o[1]);
      outv.y = pack_bf16x2(o[2], o[3]);
      outv.z = pack_bf16x2(o[4], o[5]);
      outv.w = pack_bf16x2(o[6], o[7]);
      *reinterpret_cast<uint4*>(ch.planes + (static_cast<int64_t>(r) * ch.m2 + rho[t]) * ch.ld_planes +
                                pcol) = outv;
    };
    if constexpr (kCode != 0) {
      // Straight adds and subtracts: same sums as below (start from +0, block order).
#pragma unroll
      for (int r = 0; r < kMaxRank; ++r) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = 0.f;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int c = code_coef(kCode, r, x);
          if (c == 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __fadd_rn(o[e], sv[x][e]);
          } else if (c == 3) {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __fsub_rn(o[e], sv[x][e]);
          }
        }
        store_plane(r, o);
      }
    } else {
      for (int r = 0; r < ch.plane_rank; ++r) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = 0.f;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float w = ch.plane_terms.coef[r][x];
          if (w == 0.f) continue;
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = fmaf(w, sv[x][e], o[e]);
        }
        store_plane(r, o);
      }
    }
  }
}

// The push counterpart of plane_rows32: rows [row0, row0 + 32) of each block row, columns
// [tn * 256, tn * 256 + 256) of each block column of this rank's C, read L2-hot and stored into
// the owners' slots.  256 threads: 32 16-byte vectors across, 8 rows per pass; per block row the
// 8 loads of a thread (4 passes x 2 block columns) are in flight together.
__device__ __forceinline__ void push_rows32(const PushParams& pp, int tn, int row0, int ptid) {
  const int col = tn * kBN + (ptid & 31) * 8;
  const int rsub = ptid >> 5;
  const bool col_ok[2] = {col + 8 <= pp.n2, col + 8 <= pp.n - pp.n2};
#pragma unroll 1
  for (int bi = 0; bi < 2; ++bi) {
    const int rows = bi == 0 ? pp.m2 : pp.m - pp.m2;
    uint4 q[4][2];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int r = row0 + rsub + 8 * t;
#pragma unroll
      for (int bj = 0; bj < 2; ++bj)
        if (r < rows && col_ok[bj])
          q[t][bj] = __ldcg(reinterpret_cast<const uint4*>(
              pp.c + (static_cast<int64_t>(bi) * pp.m2 + r) * pp.ldc + bj * pp.n2 + col));
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int r = row0 + rsub + 8 * t;
      if (r >= rows) continue;
      const int grow = bi * pp.m2 + r;
      const int owner = grow / pp.rows_per_owner;
      const int lrow = grow - owner * pp.rows_per_owner;
      __nv_bfloat16* dst = pp.slot[owner] + static_cast<int64_t>(lrow) * pp.n + col;
#pragma unroll
      for (int bj = 0; bj < 2; ++bj)
        if (col_ok[bj]) __stcg(reinterpret_cast<uint4*>(dst + bj * pp.n2), q[t][bj]);
    }
  }
}

// kMode: 0 plain GEMM; 1 chained (plane warps form SwiGLU + the consumer's planes behind each
// tile); 2 push (the same warps copy each finished tile to the rank that owns its rows);
// 3 fused A (the same warps form the A operand tiles from the activation matrix's blocks);
// 4 product-ahead A (the same warps of all CTAs form the A plane of the product after the one the
// MMAs are on into a global scratch, which the TMA producer reads once its chunk counter is full).
constexpr int kModePlain = 0, kModePlanes = 1, kModePush = 2, kModeFusedA = 3, kModeAheadA = 4;
// K blocks whose loads a fused-A producer thread keeps in flight in registers ahead of the block
// it is writing into shared memory.
constexpr int kFuseDepth = 2;
// Vectors of each block a plane-ahead thread keeps in flight.
constexpr int kAheadUnroll = 8;

__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <int kCtaGroup, int kMode, unsigned long long kPlaneCode = 0>
__global__ void __launch_bounds__(kMode != kModePlain ? kThreadsChain : kThreadsPlain, 1)
k_gemm(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
       const __grid_constant__ CMaps tma_c, const __grid_constant__ GemmParams p,
       const __grid_constant__ CUtensorMap tma_a2) {
  using T = Tile<kCtaGroup>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;          // swizzle atoms need 1024-byte alignment
  uint8_t* smem_gen = smem_raw + (base - raw);

  const uint32_t epi_base = base + T::kStages * T::kStageBytes;
  const uint32_t bar_base = epi_base + kEpiBufs * kEpiBytes;
  auto a_smem = [&](uint32_t s) { return base + s * T::kStageBytes; };
  auto b_smem = [&](uint32_t s) { return base + s * T::kStageBytes + T::kABytes; };
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (T::kStages + s); };
  auto acc_full_bar = [&](uint32_t s) { return bar_base + 8u * (2 * T::kStages + s); };
  auto acc_empty_bar = [&](uint32_t s) { return bar_base + 8u * (2 * T::kStages + 2 + s); };
  const uint32_t misc = bar_base + 8u * (2 * T::kStages + 4);
  volatile uint32_t* misc_gen =
      reinterpret_cast<volatile uint32_t*>(smem_gen + (misc - base));
  // misc_gen[0] = TMEM base, [1] = abort flag, [2] = units the epilogue has finished,
  // [3] = units the plane warps have finished, [4..19] = ring of plane jobs (tile index or -1)
  const uint32_t z_done_addr = misc + 8;
  const uint32_t plane_done_addr = misc + 12;
  constexpr int kJobRing = 16;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kCtaGroup == 2 ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int group_id = blockIdx.x / kCtaGroup;
  const int num_groups = gridDim.x / kCtaGroup;
  const WaitCtl ctl{&misc_gen[1], p.status};

  if (threadIdx.x == 0) {
    // A stage is full when the TMA producer's bytes have landed and, in the fused-A kernel, every
    // A-producer warp of the group has written its share of the A tile.
    constexpr uint32_t kFullArrivals = kMode == kModeFusedA ? 1u + 8u * kCtaGroup : 1u;
    for (uint32_t s = 0; s < T::kStages; ++s) {
      mbar_init(full_bar(s), kFullArrivals);
      mbar_init(empty_bar(s), 1);
    }
    for (uint32_t s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), 4 * kCtaGroup);   // one arrival per epilogue warp of the group
    }
    misc_gen[1] = 0u;
    misc_gen[2] = 0u;
    misc_gen[3] = 0u;
    fence_mbar_init();
    prefetch_tensormap(&tma_a);
    if constexpr (kMode == kModeAheadA) prefetch_tensormap(&tma_a2);
    prefetch_tensormap(&tma_b);
    prefetch_tensormap(&tma_c.m[0]);
  }
  constexpr bool kChain = kMode != kModePlain;                              // the 16-warp layout
  constexpr bool kHandoff = kMode == kModePlanes || kMode == kModePush;     // finished tiles go to the plane warps
  using R = Roles<kChain>;
  if (warp == R::kMma) {
    tmem_alloc<kCtaGroup>(misc, kTmemCols);
    tmem_relinquish<kCtaGroup>();
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {   // the peer's barriers must exist before anyone signals them
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = misc_gen[0];

  const int plane_warp = R::plane_index(warp);
  if (warp == R::kProducer) {
    // ------------------------------------------------------------ TMA producer
    // The loop body is kept to the few instructions it needs (running stage, parity and K
    // coordinate; addresses hoisted): this thread's latency is part of the stage-recycle loop.
    if (lane == 0) {
      uint32_t stage = 0, wait_parity = 1;   // parity of the "empty" phase to wait for
      // Both CTAs of a pair post their bytes on the leader's barriers.
      const uint32_t full_remote0 = kCtaGroup == 2 ? mapa_shared(full_bar(0), 0) : full_bar(0);
      for (int u = group_id; u < p.num_units; u += num_groups) {
        const UnitCoord uc = decode_unit(p, u);
        for (int s = uc.step0; s < uc.step0 + uc.nsteps; ++s) {
          const StepDesc& sd = uc.split ? p.steps_split[s] : p.steps[s];
          int a_row = sd.a_plane * p.a_plane_rows + uc.tm * T::kTileM +
                      static_cast<int>(cta_rank) * kBM;
          const int b_row = sd.b_plane * p.b_plane_rows + uc.tn * kBN +
                            static_cast<int>(cta_rank) * T::kBRows;
          int kcol = uc.kb0 * kBK;
          int a_col_off = 0;        // fused A: column of the block the single-term product reads
          bool load_a = true;
          if constexpr (kMode == kModeFusedA) {
            const int blk = p.fuse.blk[sd.a_plane][0];
            load_a = p.fuse.simt[sd.a_plane] == 0;
            a_row = (blk >> 1) * p.fuse.m2 + uc.tm * T::kTileM + static_cast<int>(cta_rank) * kBM;
            a_col_off = (blk & 1) * p.fuse.k2;
          }
          const CUtensorMap* a_map = &tma_a;
          if constexpr (kMode == kModeAheadA) {
            const int slot = p.fuse.slot[sd.a_plane];
            const int tile_row = uc.tm * T::kTileM + static_cast<int>(cta_rank) * kBM;
            if (slot < 0) {             // single block, coefficient +1: straight from the matrix
              const int blk = p.fuse.blk[sd.a_plane][0];
              a_row = (blk >> 1) * p.fuse.m2 + tile_row;
              a_col_off = (blk & 1) * p.fuse.k2;
            } else {                    // the plane the plane warps have been forming: wait until it is whole
              a_map = &tma_a2;
              a_row = slot * p.fuse.m2 + tile_row;
              global_counter_wait(p.fuse.counters + sd.a_plane, static_cast<uint32_t>(p.fuse.chunks), ctl,
                                  kCodeAhead);
              fence_proxy_async_all();  // the planes were written through the generic proxy; TMA reads them
            }
          }
          const uint32_t bytes = load_a ? T::kStageBytes : T::kBBytes;
          for (int kb = uc.kb0; kb < uc.kb1; ++kb, kcol += kBK) {
            mbar_wait(empty_bar(stage), wait_parity, ctl, kCodeProducer);
            const uint32_t sa = a_smem(stage);
            if constexpr (kCtaGroup == 1) {
              mbar_arrive_expect_tx(full_bar(stage), bytes);
              if (load_a) tma_load_2d(sa, a_map, full_bar(stage), kcol + a_col_off, a_row);
              tma_load_2d(sa + T::kABytes, &tma_b, full_bar(stage), kcol, b_row);
            } else {
              if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * bytes);
              const uint32_t bar = full_remote0 + 8u * stage;
              if (load_a) tma_load_2d_pair(sa, a_map, bar, kcol + a_col_off, a_row);
              tma_load_2d_pair(sa + T::kABytes, &tma_b, bar, kcol, b_row);
            }
            if (++stage == T::kStages) {
              stage = 0;
              wait_parity ^= 1u;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == R::kMma) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM * kCtaGroup, kBN);
      uint32_t stage = 0, parity = 0, acc_it = 0;
      // Operand descriptors of stage 0; a stage further on adds its byte offset >> 4 to the
      // address field (stages are 1024-byte aligned, so nothing carries out of the field).
      const uint64_t adesc0 = make_kmajor_sw128_desc(a_smem(0));
      const uint64_t bdesc0 = make_kmajor_sw128_desc(b_smem(0));
      for (int u = group_id; u < p.num_units; u += num_groups) {
        const UnitCoord uc = decode_unit(p, u);
        for (int s = uc.step0; s < uc.step0 + uc.nsteps; ++s, ++acc_it) {
          const uint32_t as = acc_it & 1u;
          const uint32_t aphase = (acc_it >> 1) & 1u;
          mbar_wait(acc_empty_bar(as), aphase ^ 1u, ctl, kCodeMmaAcc);
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + as * kBN;
          uint32_t accumulate = (uc.split || p.steps[s].clear) ? 0u : 1u;
          for (int kb = uc.kb0; kb < uc.kb1; ++kb) {
            mbar_wait(full_bar(stage), parity, ctl, kCodeMmaFull);
            tcgen05_fence_after();
            const uint64_t soff = static_cast<uint64_t>(stage * (T::kStageBytes >> 4));
            const uint64_t adesc = adesc0 + soff;
            const uint64_t bdesc = bdesc0 + soff;
            // +32 bytes per K=16 slice inside the 128-byte swizzle row
            umma_bf16<kCtaGroup>(d_tmem, adesc, bdesc, idesc, accumulate);
#pragma unroll
            for (int k = 1; k < kBK / kUmmaK; ++k)
              umma_bf16<kCtaGroup>(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, 1u);
            accumulate = 1u;
            umma_commit<kCtaGroup>(empty_bar(stage));   // frees the stage in every CTA of the group
            if (++stage == T::kStages) {
              stage = 0;
              parity ^= 1u;
            }
          }
          umma_commit<kCtaGroup>(acc_full_bar(as));
        }
      }
    }
    __syncwarp();
  } else if (R::is_epilogue(warp)) {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;                 // TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;          // row inside the CTA's 128-row tile
    const bool issuer = warp == R::kEpiIssuer && lane == 0;
    const uint32_t acc_empty_remote =
        kCtaGroup == 2 ? mapa_shared(acc_empty_bar(0), 0) : acc_empty_bar(0);
    uint32_t acc_it = 0, epi_it = 0, units_done = 0;
    for (int u = group_id; u < p.num_units; u += num_groups) {
      const UnitCoord uc = decode_unit(p, u);
      const int row0 = uc.tm * T::kTileM + static_cast<int>(cta_rank) * kBM;
      const int col0 = uc.tn * kBN;
      for (int s = uc.step0; s < uc.step0 + uc.nsteps; ++s, ++acc_it) {
        const uint32_t as = acc_it & 1u;
        const uint32_t aphase = (acc_it >> 1) & 1u;
        mbar_wait(acc_full_bar(as), aphase, ctl, kCodeEpilogue);
        tcgen05_fence_after();
        const StepDesc& sd = uc.split ? p.steps_split[s] : p.steps[s];
        for (int g = 0; g < sd.ngroups; ++g) {
          // +1 and -1 (every shipped table) need no multiplication: rounding to bf16 is symmetric, so
          // -1 is a flip of the packed sign bits after the conversion.  Same bits, half the arithmetic.
          const int coeff_i = sd.group[g].coeff;
          const float coeff = static_cast<float>(coeff_i);
#pragma unroll 1
          for (int sub = 0; sub < kBN / kEpiCols; ++sub, ++epi_it) {
            uint32_t r0[32], r1[32];
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   as * kBN + sub * kEpiCols;
            tmem_ld_32x32(taddr, r0);
            tmem_ld_32x32(taddr + 32, r1);
            tmem_ld_wait();
            uint32_t pk[32];
            if (coeff_i == 1 || coeff_i == -1) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                pk[j] = pack_bf16x2(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                pk[16 + j] = pack_bf16x2(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
              }
              if (coeff_i < 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) pk[j] ^= 0x80008000u;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                pk[j] = pack_bf16x2(coeff * __uint_as_float(r0[2 * j]),
                                    coeff * __uint_as_float(r0[2 * j + 1]));
                pk[16 + j] = pack_bf16x2(coeff * __uint_as_float(r1[2 * j]),
                                         coeff * __uint_as_float(r1[2 * j + 1]));
              }
            }
            const uint32_t buf = epi_base + (epi_it & 1u) * kEpiBytes;
            // The bulk copy issued two sub-tiles ago read this buffer; it must be done.
            if (issuer) bulk_wait_group_read<1>();
            __syncwarp();
            named_bar_sync(1, 128);
            const uint32_t row_addr = buf + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              st_shared_v4(row_addr + (((c ^ (row & 7)) << 4)), pk[4 * c], pk[4 * c + 1],
                           pk[4 * c + 2], pk[4 * c + 3]);
            fence_proxy_async_shared();
            named_bar_sync(1, 128);
            if (issuer) {
              for (int d = 0; d < sd.group[g].ndest; ++d) {
                const EpiDest dst = sd.group[g].dest[d];
                const CUtensorMap* cm = &tma_c.m[dst.bi * 2 + dst.bj];
#pragma unroll
                for (int j = 0; j < kBM / kEpiBoxRows; ++j) {
                  const uint32_t src = buf + j * kEpiBoxRows * 128;
                  if (dst.first)
                    tma_store_2d(cm, src, col0 + sub * kEpiCols, row0 + j * kEpiBoxRows);
                  else
                    tma_reduce_add_2d(cm, src, col0 + sub * kEpiCols, row0 + j * kEpiBoxRows);
                }
              }
              bulk_commit_group();
            }
            __syncwarp();
          }
        }
        // This warp's reads of the stage are complete: hand it back to the MMA issuer.
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtaGroup == 1)
            mbar_arrive(acc_empty_bar(as));
          else
            mbar_arrive_cluster(acc_empty_remote + 8u * as);
        }
      }
      if constexpr (kHandoff) {
        // Hand the unit to the plane warps.  A whole tile's C blocks are final once this CTA's
        // bulk copies have landed (single writer), so its plane job runs here, under the next
        // tile's MMAs.  A tail tile is written by several CTAs and is final only when the kernel
        // ends: its planes are formed by k_tail_planes, launched behind this kernel.
        if (issuer) {
          int job = -1;
          if (uc.tail < 0) {
            bulk_wait_group<0>();
            fence_proxy_async_all();
            job = uc.tile;
          }
          // the ring entry being overwritten must have been consumed
          if (units_done >= kJobRing - 1)
            counter_wait(plane_done_addr, units_done - (kJobRing - 2), ctl, kCodePlane);
          misc_gen[4 + (units_done % kJobRing)] = static_cast<uint32_t>(job);
          st_release_shared(z_done_addr, ++units_done);
        }
        __syncwarp();
      }
    }
    if (issuer) bulk_wait_group<0>();
    __syncwarp();
  } else if constexpr (kMode == kModeFusedA) {
    if (plane_warp >= 0) {
      // ------------------------------------------------------- A-operand producer warps
      // 256 threads form the 128 x 64 A tile of every K block of every step this CTA walks:
      // thread (rsub, vec) owns the 16-byte vector `vec` of rows rsub + 32 j (j = 0..3).  The
      // blocks' vectors are loaded kFuseDepth K blocks ahead into registers, combined with one
      // packed bf16 add or subtract (for two terms this is the fp32 sum rounded once: the exact sum
      // of two bf16 values whose exponents differ by less than 16 fits fp32, and beyond that the
      // smaller term cannot move the rounding of the larger), written with the 128-byte swizzle
      // the MMA descriptors expect, fenced towards the async proxy, and the warp arrives on the
      // stage's full barrier.  A step whose product reads a single block with coefficient +1 is
      // loaded by the TMA producer instead; these warps then only wait and arrive.
      const FuseParams& fp = p.fuse;
      const int ptid = plane_warp * 32 + lane;
      const int vec = ptid & 7;
      const int rsub = ptid >> 3;
      const uint32_t sw_off = static_cast<uint32_t>(rsub) * 128u +
                              (static_cast<uint32_t>(vec ^ (rsub & 7)) << 4);
      const uint32_t full_remote0 = kCtaGroup == 2 ? mapa_shared(full_bar(0), 0) : full_bar(0);
      constexpr uint32_t kNone = 0xffffffffu;

      // Walk of the (unit, step, K block) sequence, kFuseDepth items ahead of the writes.
      int w_u = group_id, w_s = 0, w_s_end = 0, w_kb = 0, w_kb_end = 0;
      bool w_valid = false, w_split = false;
      UnitCoord w_uc = {};
      const __nv_bfloat16* w_ptr[2] = {nullptr, nullptr};
      // bit 0: the step goes through these warps; bits 1-2: its terms; bits 3-4: term negated;
      // bit 8 + 4 t + j: vector j of term t lies past the last row of the matrix and reads as zero
      uint32_t w_meta = 0;
      auto w_begin_step = [&]() {
        const StepDesc& sd = w_split ? p.steps_split[w_s] : p.steps[w_s];
        const int r = sd.a_plane;
        const int nterm = fp.nterm[r];
        w_meta = (fp.simt[r] ? 1u : 0u) | (static_cast<uint32_t>(nterm) << 1) |
                 (fp.neg[r][0] ? 8u : 0u) | (fp.neg[r][1] ? 16u : 0u);
        const int row_in_block = w_uc.tm * T::kTileM + static_cast<int>(cta_rank) * kBM + rsub;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int blk = fp.blk[r][t < nterm ? t : 0];
          const int64_t grow = static_cast<int64_t>(blk >> 1) * fp.m2 + row_in_block;
          w_ptr[t] = fp.a + grow * fp.lda + static_cast<int64_t>(blk & 1) * fp.k2 +
                     static_cast<int64_t>(w_kb) * kBK + vec * 8;
          // Rows past the end of the matrix must not be read.  (Rows past the end of a block
          // row but inside the matrix feed accumulator rows that the clipped C maps never store.)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (t < nterm && grow + 32 * j >= fp.m) w_meta |= 1u << (8 + 4 * t + j);
        }
      };
      auto w_begin_unit = [&]() {
        w_valid = w_u < p.num_units;
        if (!w_valid) return;
        w_uc = decode_unit(p, w_u);
        w_split = w_uc.split != 0;
        w_s = w_uc.step0;
        w_s_end = w_uc.step0 + w_uc.nsteps;
        w_kb = w_uc.kb0;
        w_kb_end = w_uc.kb1;
        w_begin_step();
      };
      auto w_advance = [&]() {
        w_ptr[0] += kBK;
        w_ptr[1] += kBK;
        if (++w_kb < w_kb_end) return;
        w_kb = w_uc.kb0;
        if (++w_s < w_s_end) {
          w_begin_step();
          return;
        }
        w_u += num_groups;
        w_begin_unit();
      };
      auto w_issue = [&](uint4 (&dst)[2][4]) -> uint32_t {
        if (!w_valid) return kNone;
        const uint32_t meta = w_meta;
        if (meta & 1u) {
          const int nterm = static_cast<int>((meta >> 1) & 3u);
#pragma unroll
          for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (t < nterm && ((meta >> (8 + 4 * t + j)) & 1u) == 0u)
                dst[t][j] = __ldcg(reinterpret_cast<const uint4*>(w_ptr[t] + static_cast<int64_t>(32 * j) * fp.lda));
              else
                dst[t][j] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        w_advance();
        return meta;
      };

      uint4 buf[kFuseDepth][2][4];
      uint32_t meta[kFuseDepth];
      w_begin_unit();
#pragma unroll
      for (int d = 0; d < kFuseDepth; ++d) meta[d] = w_issue(buf[d]);
      uint32_t stage = 0, wait_parity = 1;
      bool more = true;
      while (more) {
#pragma unroll
        for (int d = 0; d < kFuseDepth; ++d) {
          if (meta[d] == kNone) {
            more = false;
            break;
          }
          if (lane == 0) mbar_wait(empty_bar(stage), wait_parity, ctl, kCodePlane);
          __syncwarp();
          if (meta[d] & 1u) {
            const uint32_t dst = a_smem(stage) + sw_off;
            const bool two = ((meta[d] >> 1) & 3u) == 2u;
            const bool neg0 = (meta[d] & 8u) != 0u, neg1 = (meta[d] & 16u) != 0u;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 x = buf[d][0][j];
              const uint4 y = buf[d][1][j];
              if (neg0) {      // -x (+- y): flip the signs, exact
                x.x ^= 0x80008000u, x.y ^= 0x80008000u, x.z ^= 0x80008000u, x.w ^= 0x80008000u;
              }
              if (two) {
                if (neg1) {
                  x.x = bf16x2_sub(x.x, y.x), x.y = bf16x2_sub(x.y, y.y);
                  x.z = bf16x2_sub(x.z, y.z), x.w = bf16x2_sub(x.w, y.w);
                } else {
                  x.x = bf16x2_add(x.x, y.x), x.y = bf16x2_add(x.y, y.y);
                  x.z = bf16x2_add(x.z, y.z), x.w = bf16x2_add(x.w, y.w);
                }
              }
              st_shared_v4(dst + static_cast<uint32_t>(j) * (32u * 128u), x.x, x.y, x.z, x.w);
            }
            fence_proxy_async_shared();
          }
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtaGroup == 1)
              mbar_arrive(full_bar(stage));
            else
              mbar_arrive_cluster(full_remote0 + 8u * stage);
          }
          if (++stage == T::kStages) {
            stage = 0;
            wait_parity ^= 1u;
          }
          meta[d] = w_issue(buf[d]);
        }
      }
    }
  } else if constexpr (kMode == kModeAheadA) {
    if (plane_warp >= 0) {
      // ----------------------------------------------- plane warps, one product ahead
      // The two-term products' A planes, in the order the steps need them.  A plane is cut
      // into chunks of `chunk_rows` rows; chunk c belongs to CTA c mod gridDim.x.  These warps
      // never wait for anything, so every counter fills whatever the MMA side is doing.
      const FuseParams& fp = p.fuse;
      const int ptid = plane_warp * 32 + lane;
      const int nvec = fp.k2 >> 3;
      for (int o = 0; o < fp.nslots; ++o) {
        const int r = fp.order[o];
        const int b0 = fp.blk[r][0], b1 = fp.blk[r][1];
        const bool neg0 = fp.neg[r][0] != 0, neg1 = fp.neg[r][1] != 0;
        const __nv_bfloat16* src0 = fp.a + static_cast<int64_t>(b0 >> 1) * fp.m2 * fp.lda +
                                    static_cast<int64_t>(b0 & 1) * fp.k2;
        const __nv_bfloat16* src1 = fp.a + static_cast<int64_t>(b1 >> 1) * fp.m2 * fp.lda +
                                    static_cast<int64_t>(b1 & 1) * fp.k2;
        const int rows0 = (b0 >> 1) ? fp.m - fp.m2 : fp.m2;     // rows block row b >> 1 really has
        const int rows1 = (b1 >> 1) ? fp.m - fp.m2 : fp.m2;
        __nv_bfloat16* dst = fp.scratch + static_cast<int64_t>(fp.slot[r]) * fp.m2 * fp.k2;
        for (int c = static_cast<int>(blockIdx.x); c < fp.chunks; c += static_cast<int>(gridDim.x)) {
          // The chunk's rows x vectors as one index space, kAheadUnroll vectors of each block in
          // flight per thread (the loads' round trip, not their issue rate, sets the pace).
          const int row0 = c * fp.chunk_rows;
          const int total = (min(row0 + fp.chunk_rows, fp.m2) - row0) * nvec;
          for (int base = ptid; base < total; base += kPlaneThreads * kAheadUnroll) {
            uint4 x[kAheadUnroll], y[kAheadUnroll];
            int64_t doff[kAheadUnroll];
#pragma unroll
            for (int u = 0; u < kAheadUnroll; ++u) {
              const int e = base + u * kPlaneThreads;
              const int row = row0 + e / nvec;
              const int v = e - (e / nvec) * nvec;
              const bool in = e < total;
              doff[u] = in ? static_cast<int64_t>(row) * fp.k2 + v * 8 : -1;
              x[u] = (in && row < rows0)
                         ? __ldcs(reinterpret_cast<const uint4*>(src0 + static_cast<int64_t>(row) * fp.lda) + v)
                         : make_uint4(0u, 0u, 0u, 0u);
              y[u] = (in && row < rows1)
                         ? __ldcs(reinterpret_cast<const uint4*>(src1 + static_cast<int64_t>(row) * fp.lda) + v)
                         : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < kAheadUnroll; ++u) {
              uint4 q = x[u];
              if (neg0) q.x ^= 0x80008000u, q.y ^= 0x80008000u, q.z ^= 0x80008000u, q.w ^= 0x80008000u;
              if (neg1) {
                q.x = bf16x2_sub(q.x, y[u].x), q.y = bf16x2_sub(q.y, y[u].y);
                q.z = bf16x2_sub(q.z, y[u].z), q.w = bf16x2_sub(q.w, y[u].w);
              } else {
                q.x = bf16x2_add(q.x, y[u].x), q.y = bf16x2_add(q.y, y[u].y);
                q.z = bf16x2_add(q.z, y[u].z), q.w = bf16x2_add(q.w, y[u].w);
              }
              if (doff[u] >= 0) *reinterpret_cast<uint4*>(dst + doff[u]) = q;
            }
          }
          // Publish the chunk: every writer orders its stores before the async proxy's later
          // reads and makes them visible GPU-wide, then one thread counts the chunk.
          fence_proxy_async_all();
          __threadfence();
          named_bar_sync(2, kPlaneThreads);
          if (ptid == 0) atomicAdd(fp.counters + r, 1u);
        }
      }
    }
  } else if constexpr (kChain) {
    if (plane_warp >= 0) {
    // ------------------------------------------------------------- plane warps
    const ChainParams& ch = p.chain;
    const int ptid = plane_warp * 32 + lane;
    const int tiles_total = p.tiles_m * p.tiles_n;
    const int64_t clear_stride =
        static_cast<int64_t>(gridDim.x) * kPlaneThreads * ch.iters_max;
    auto clear_share = [&](int t) {
      if (ch.preclear == nullptr) return;
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      if (ch.preload == nullptr) {
        for (int64_t i = (static_cast<int64_t>(t) * gridDim.x + blockIdx.x) * kPlaneThreads + ptid;
             i < ch.preclear_vecs; i += clear_stride)
          ch.preclear[i] = zero;
      } else {
        // The consumer adds its contributions onto the residual stream: start from that.
        for (int64_t i = (static_cast<int64_t>(t) * gridDim.x + blockIdx.x) * kPlaneThreads + ptid;
             i < ch.preclear_vecs; i += clear_stride)
          ch.preclear[i] = __ldcs(ch.preload + i);
      }
    };
    uint32_t seq = 0;
    for (int u = group_id; u < p.num_units; u += num_groups, ++seq) {
      clear_share(static_cast<int>(seq));
      if (lane == 0) counter_wait(z_done_addr, seq + 1, ctl, kCodePlane);   // one poller per warp
      __syncwarp();
      const int job = static_cast<int>(misc_gen[4 + (seq % kJobRing)]);
      // A job names a tile whose four C blocks are final.  (After a run-out wait the ring may
      // hold anything: only a valid tile index is ever acted on.)
      if (job >= 0 && job < tiles_total && misc_gen[1] == 0u) {
        fence_proxy_async_all();
        int tm, tn;
        tile_coord(p, job, tm, tn);
        const int row_base = tm * T::kTileM + static_cast<int>(cta_rank) * kBM;
        if constexpr (kMode == kModePush) {
#pragma unroll 1
          for (int step = 0; step < kBM / 32; ++step) push_rows32(p.push, tn, row_base + step * 32, ptid);
        } else {
#pragma unroll 1
          for (int step = 0; step < kBM / 32; ++step)
            plane_rows32<kPlaneCode>(ch, tn, row_base + step * 32, ptid);
        }
      }
      // every plane thread has read its ring entry: the epilogue may reuse it
      named_bar_sync(2, kPlaneThreads);
      if (ptid == 0) st_release_shared(plane_done_addr, seq + 1);
    }
    for (int t = static_cast<int>(seq); t < ch.iters_max; ++t) clear_share(t);
    }   // plane warps (the two spare warps of the block go straight to the teardown)
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (misc_gen[1] != 0u && warp == R::kProducer) {
    // A wait ran out somewhere: loads may still be in flight towards this CTA's
    // shared memory.  Give them time to land before the CTA goes away.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {   // neither CTA may leave while its peer can still signal it
    cluster_arrive();
    cluster_wait();
  }
  if (warp == R::kMma) {
    tcgen05_fence_after();
    tmem_dealloc<kCtaGroup>(tmem_base, kTmemCols);
  }
}

// Zero the C blocks of the tail tiles of a hybrid launch (their products arrive as
// reduce-adds from several CTAs).  grid = (tail tiles, 4 blocks, 4 row quarters), 256 threads.
struct ZeroArgs {
  __nv_bfloat16* c;
  int64_t ldc;
  int32_t m, n, m2, n2, tile_m;
};
__global__ void __launch_bounds__(256)
k_zero_tail_tiles(const __grid_constant__ GemmParams p, const ZeroArgs z) {
  int tm, tn;
  tile_coord(p, p.main_tiles + static_cast<int>(blockIdx.x), tm, tn);
  const int bi = blockIdx.y >> 1, bj = blockIdx.y & 1;
  const int rows = bi == 0 ? z.m2 : z.m - z.m2;
  const int cols = bj == 0 ? z.n2 : z.n - z.n2;
  const int quarter = z.tile_m / 4;
  const int r0 = tm * z.tile_m + static_cast<int>(blockIdx.z) * quarter;
  const int r1 = min(r0 + quarter, rows);
  const int c1 = min(tn * kBN + kBN, cols);
  __nv_bfloat16* base = z.c + static_cast<int64_t>(bi) * z.m2 * z.ldc + static_cast<int64_t>(bj) * z.n2;
  const int col = tn * kBN + (threadIdx.x & 31) * 8;
  for (int row = r0 + (threadIdx.x >> 5); row < r1; row += 8) {
    __nv_bfloat16* ptr = base + static_cast<int64_t>(row) * z.ldc + col;
    if (col + 8 <= c1) {
      *reinterpret_cast<uint4*>(ptr) = make_uint4(0u, 0u, 0u, 0u);
    } else {
      for (int e = 0; col + e < c1; ++e) ptr[e] = __float2bfloat16(0.f);
    }
  }
}

// SwiGLU + consumer planes (or the tensor-parallel push) of the tail tiles of a chained hybrid
// launch, behind the GEMM kernel (their C blocks are sums over several CTAs and final only when
// it ends).  One CTA per 32 rows
// of a tile: grid = tail tiles * tile_m / 32, 256 threads.
template <unsigned long long kPlaneCode>
__global__ void __launch_bounds__(kPlaneThreads)
k_tail_planes(const __grid_constant__ GemmParams p, const int tile_m) {
  const int chunks = tile_m / 32;
  const int n = static_cast<int>(blockIdx.x) / chunks;
  const int c = static_cast<int>(blockIdx.x) - n * chunks;
  int tm, tn;
  tile_coord(p, p.main_tiles + n, tm, tn);
  if (p.push.world > 0)
    push_rows32(p.push, tn, tm * tile_m + c * 32, static_cast<int>(threadIdx.x));
  else
    plane_rows32<kPlaneCode>(p.chain, tn, tm * tile_m + c * 32, static_cast<int>(threadIdx.x));
}

// ============================================================== host side
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

// bf16 row-major (outer x inner) matrix, 128-byte swizzled boxes of box_outer x 64.
int make_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld,
             int box_outer, const char* what) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return fail(LCG_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(LCG_ERR_MISALIGNED, "%s: base address must be 16-byte aligned", what);
  if (ld % 8 != 0)
    return fail(LCG_ERR_MISALIGNED, "%s: leading dimension %lld must be a multiple of 8 elements", what,
                (long long)ld);
  if (inner < 1 || outer < 1) return fail(LCG_ERR_UNSUPPORTED_SHAPE, "%s: empty extent", what);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_outer)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(LCG_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return LCG_OK;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2)
      sms = 148;
  }
  return sms;
}

// Tile rows kept open at once: the divisor-free version of "minimise a + groups / a".
int pick_group_m(int tiles_m, int groups) {
  int best = 1;
  double best_cost = 1e30;
  for (int a = 1; a <= tiles_m; ++a) {
    if (tiles_m % a != 0) continue;
    const double cost = a + static_cast<double>(groups) / a;
    if (cost < best_cost) {
      best_cost = cost;
      best = a;
    }
  }
  return best;
}

template <int kCtaGroup, int kMode, unsigned long long kPlaneCode = 0>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CMaps& mc, GemmParams& p,
           cudaStream_t stream, const CUtensorMap* ma2 = nullptr) {
  using T = Tile<kCtaGroup>;
  constexpr bool kChain = kMode != kModePlain;
  auto kern = k_gemm<kCtaGroup, kMode, kPlaneCode>;
  static bool configured[64] = {};   // per device: the attribute belongs to the device's context
  int dev = 0;
  LCG_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    LCG_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  int max_groups = sm_count() / kCtaGroup;
  if (p.max_groups > 0 && p.max_groups < max_groups) max_groups = p.max_groups;
  const int groups = p.num_units < max_groups ? p.num_units : max_groups;
  if (kChain) p.chain.iters_max = (p.num_units + groups - 1) / groups;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(groups * kCtaGroup));
  cfg.blockDim = dim3(kChain ? kThreadsChain : kThreadsPlain);
  cfg.dynamicSmemBytes = T::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtaGroup;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  LCG_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, p, ma2 != nullptr ? *ma2 : ma));
  count_launch();
  return LCG_OK;
}

int resolve_group(int cta_group) {
  if (cta_group == LCG_CTA_GROUP_DEFAULT) return 2;
  return cta_group;
}

struct R7Geometry {
  int64_t m2, n2, k2p;
};

int r7_geometry(int64_t M, int64_t N, int64_t K, R7Geometry* g) {
  if (M < 2 || N < 2 || K < 2)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "rank-7 GEMM needs M, N, K >= 2");
  int64_t k2;
  lcg_plane_geometry(M, K, 1, &g->m2, &k2, &g->k2p);
  lcg_plane_geometry(N, K, 8, &g->n2, nullptr, nullptr);
  if (N - g->n2 < 1)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "N=%lld leaves the second column block empty", (long long)N);
  if (7 * g->m2 > 0x7fffffffLL || 7 * g->n2 > 0x7fffffffLL)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "operand too tall");
  return LCG_OK;
}

// The unit list of a launch (see GemmParams) for `tiles` tiles on `groups` CTA groups.
void plan_units(int rank, int tiles, int groups, int k_blocks, int schedule, GemmParams* p) {
  p->main_tiles = tiles;
  p->tail_tiles = 0;
  p->ksplit = 1;
  p->zero_tail = 0;
  if (schedule == LCG_SCHEDULE_RANK_SPLIT) {
    p->main_tiles = 0;
    p->tail_tiles = tiles;
  } else if (schedule == LCG_SCHEDULE_HYBRID) {
    // Whole waves walk all products per tile; the last partial wave is split by product when
    // that shortens it: ceil(rank * tail / groups) single steps against `rank` steps.
    const int tail = tiles % groups;
    const int split_steps = (rank * tail + groups - 1) / groups;
    if (tail > 0 && split_steps <= rank - 2) {
      p->main_tiles = tiles - tail;
      p->tail_tiles = tail;
      p->zero_tail = 1;
    }
  }
  // Single-product units fill whole rounds of the CTA groups over the full K; the units of the
  // last partial round are cut into `ksplit` K ranges so that the round shortens to
  // ceil(rest * ksplit / groups) / ksplit of a unit (each extra range costs an epilogue).
  const int prod_units = rank * p->tail_tiles;
  p->full_units = prod_units;
  p->split_units = 0;
  const int rest = prod_units % groups;
  if (rest > 0) {
    int best_f = 1;
    double best = 1.0;
    for (int f = 2; f <= 8; ++f) {
      if (k_blocks / f < 8) break;
      const double cost = static_cast<double>((rest * f + groups - 1) / groups) / f + 0.02 * f;
      if (cost < best - 0.05) {
        best = cost;
        best_f = f;
      }
    }
    if (best_f > 1) {
      p->ksplit = best_f;
      p->full_units = prod_units - rest;
      p->split_units = rest;
    }
  }
  p->num_units = p->main_tiles + p->full_units + p->split_units * p->ksplit;
}

int fill_r7(const lcg_scheme* scheme, const void* a_planes, int64_t ld_a, const void* b_planes,
            int64_t ld_b, void* c, int64_t ldc, int64_t M, int64_t N, const R7Geometry& g,
            int schedule, int cta_group, CUtensorMap* ma, CUtensorMap* mb, CMaps* mc,
            GemmParams* p, int tm_begin = 0, int tm_end = -1, int max_groups = 0,
            int64_t a_matrix_cols = 0) {
  const int tile_m = kBM * cta_group;
  // a_matrix_cols > 0: `a_planes` is the (M, K) activation matrix itself (fused A producer).
  if (a_matrix_cols > 0) {
    if (int e = make_map(ma, a_planes, a_matrix_cols, M, ld_a, kBM, "A")) return e;
  } else if (int e = make_map(ma, a_planes, g.k2p, scheme->rank * g.m2, ld_a, kBM, "A planes")) {
    return e;
  }
  if (int e = make_map(mb, b_planes, g.k2p, scheme->rank * g.n2, ld_b, kBN / cta_group, "B planes"))
    return e;
  for (int bi = 0; bi < 2; ++bi)
    for (int bj = 0; bj < 2; ++bj) {
      const int64_t rows = bi == 0 ? g.m2 : M - g.m2;
      const int64_t cols = bj == 0 ? g.n2 : N - g.n2;
      const __nv_bfloat16* blk =
          static_cast<const __nv_bfloat16*>(c) + bi * g.m2 * ldc + bj * g.n2;
      if (int e = make_map(&mc->m[bi * 2 + bj], blk, cols, rows, ldc, kEpiBoxRows, "C block")) return e;
    }
  std::memset(p, 0, sizeof(*p));
  for (int t = 0; t < scheme->rank; ++t) {
    p->steps[t] = scheme->all_ranks[t];
    p->steps_split[t] = scheme->rank_split[t];
  }
  p->steps_per_unit = scheme->rank;
  const int tiles_m_all = static_cast<int>((g.m2 + tile_m - 1) / tile_m);
  if (tm_end < 0) tm_end = tiles_m_all;
  if (tm_begin < 0 || tm_begin >= tm_end || tm_end > tiles_m_all)
    return fail(LCG_ERR_BAD_ARG, "tile-row slab [%d, %d) outside [0, %d)", tm_begin, tm_end, tiles_m_all);
  p->tm_base = tm_begin;
  p->tiles_m = tm_end - tm_begin;
  p->tiles_n = static_cast<int>((g.n2 + kBN - 1) / kBN);
  int groups = sm_count() / cta_group;
  if (max_groups > 0 && max_groups < groups) groups = max_groups;
  p->max_groups = max_groups;
  p->group_m = pick_group_m(p->tiles_m, groups);
  p->k_blocks = static_cast<int>(g.k2p / kBK);
  plan_units(scheme->rank, p->tiles_m * p->tiles_n, groups, p->k_blocks, schedule, p);
  p->num_units = p->main_tiles + p->full_units + p->split_units * p->ksplit;
  p->a_plane_rows = static_cast<int>(g.m2);
  p->b_plane_rows = static_cast<int>(g.n2);
  return LCG_OK;
}

// The C blocks of the tail tiles receive reduce-adds only: clear them first, on the stream.
int zero_tail_tiles(const GemmParams& p, void* c, int64_t ldc, int64_t M, int64_t N,
                    const R7Geometry& g, int cta_group, cudaStream_t stream) {
  if (p.tail_tiles == 0 || !p.zero_tail) return LCG_OK;
  ZeroArgs z;
  z.c = static_cast<__nv_bfloat16*>(c);
  z.ldc = ldc;
  z.m = static_cast<int32_t>(M);
  z.n = static_cast<int32_t>(N);
  z.m2 = static_cast<int32_t>(g.m2);
  z.n2 = static_cast<int32_t>(g.n2);
  z.tile_m = kBM * cta_group;
  k_zero_tail_tiles<<<dim3(static_cast<unsigned>(p.tail_tiles), 4, 4), 256, 0, stream>>>(p, z);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

}  // namespace
}  // namespace lcg

using namespace lcg;

extern "C" int lcg_gemm_dense(const void* a, int64_t lda, const void* b, int64_t ldb, void* c,
                              int64_t ldc, int64_t M, int64_t N, int64_t K, int cta_group,
                              int32_t* status, void* stream) {
  if (!a || !b || !c) return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (M < 1 || N < 1 || K < 8 || K % 8 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "dense GEMM needs K %% 8 == 0, got M=%lld N=%lld K=%lld",
                (long long)M, (long long)N, (long long)K);
  if (lda < K || ldb < K || ldc < N) return fail(LCG_ERR_BAD_ARG, "leading dimension below extent");
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  CUtensorMap ma, mb;
  CMaps mc;
  if (int e = make_map(&ma, a, K, M, lda, kBM, "A")) return e;
  if (int e = make_map(&mb, b, K, N, ldb, kBN / cta_group, "B")) return e;
  if (int e = make_map(&mc.m[0], c, N, M, ldc, kEpiBoxRows, "C")) return e;
  mc.m[1] = mc.m[2] = mc.m[3] = mc.m[0];
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  StepDesc& st = p.steps[0];
  st.clear = 1;
  st.ngroups = 1;
  st.group[0].coeff = 1;
  st.group[0].ndest = 1;
  st.group[0].dest[0].first = 1;
  const int tile_m = kBM * cta_group;
  p.steps_per_unit = 1;
  p.tiles_m = static_cast<int>((M + tile_m - 1) / tile_m);
  p.tiles_n = static_cast<int>((N + kBN - 1) / kBN);
  p.group_m = pick_group_m(p.tiles_m, sm_count() / cta_group);
  p.num_units = p.tiles_m * p.tiles_n;
  p.main_tiles = p.num_units;
  p.k_blocks = static_cast<int>((K + kBK - 1) / kBK);
  p.status = status;
  auto st_ = static_cast<cudaStream_t>(stream);
  return cta_group == 1 ? launch<1, kModePlain>(ma, mb, mc, p, st_) : launch<2, kModePlain>(ma, mb, mc, p, st_);
}

extern "C" int lcg_gemm_r7(const lcg_scheme_t* scheme, const void* a_planes, int64_t ld_a,
                           const void* b_planes, int64_t ld_b, void* c, int64_t ldc, int64_t M,
                           int64_t N, int64_t K, int schedule, int cta_group, int32_t* status,
                           void* stream) {
  if (!scheme || !a_planes || !b_planes || !c) return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (schedule != LCG_SCHEDULE_ALL_RANKS && schedule != LCG_SCHEDULE_RANK_SPLIT &&
      schedule != LCG_SCHEDULE_HYBRID)
    return fail(LCG_ERR_BAD_ARG, "unknown schedule %d", schedule);
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  R7Geometry g;
  if (int e = r7_geometry(M, N, K, &g)) return e;
  if (ldc < N) return fail(LCG_ERR_BAD_ARG, "ldc below N");
  if (ld_a < g.k2p || ld_b < g.k2p) return fail(LCG_ERR_BAD_ARG, "plane leading dimension below K2p");
  CUtensorMap ma, mb;
  CMaps mc;
  GemmParams p;
  if (int e = fill_r7(scheme, a_planes, ld_a, b_planes, ld_b, c, ldc, M, N, g, schedule, cta_group,
                      &ma, &mb, &mc, &p))
    return e;
  p.status = status;
  auto st_ = static_cast<cudaStream_t>(stream);
  if (int e = zero_tail_tiles(p, c, ldc, M, N, g, cta_group, st_)) return e;
  return cta_group == 1 ? launch<1, kModePlain>(ma, mb, mc, p, st_) : launch<2, kModePlain>(ma, mb, mc, p, st_);
}

// Which blocks of A each product reads, for the fused A producer.  Fails for a table with more
// than two terms in a row (the producer warps hold two blocks' vectors per K block).
static int fill_fuse(const lcg_scheme* scheme, const void* a, int64_t lda, int64_t M, int64_t K,
                     const R7Geometry& g, FuseParams* f) {
  std::memset(f, 0, sizeof(*f));
  f->a = static_cast<const __nv_bfloat16*>(a);
  f->lda = lda;
  f->m = static_cast<int32_t>(M);
  f->m2 = static_cast<int32_t>(g.m2);
  f->k2 = static_cast<int32_t>(K / 2);
  for (int r = 0; r < scheme->rank; ++r) {
    int n = 0;
    for (int x = 0; x < 4; ++x) {
      const int c = scheme->a[r][x];
      if (c == 0) continue;
      if ((c != 1 && c != -1) || n == 2)
        return fail(LCG_ERR_SCHEME,
                    "the fused A producer needs A-side rows with one or two +-1 terms; product %d of "
                    "this scheme has more (use lcg_a_planes + lcg_gemm_r7)", r);
      f->blk[r][n] = static_cast<int8_t>(x);
      f->neg[r][n] = c < 0;
      ++n;
    }
    if (n == 0) return fail(LCG_ERR_SCHEME, "product %d reads no block of A", r);
    f->nterm[r] = static_cast<int8_t>(n);
    f->simt[r] = !(n == 1 && !f->neg[r][0]);
  }
  return LCG_OK;
}

extern "C" int lcg_gemm_r7_fused_supported(const lcg_scheme_t* scheme, int64_t M, int64_t N, int64_t K) {
  if (!scheme || M < 2 || N < 2 || K < 128 || K % 128 != 0) return 0;
  for (int r = 0; r < scheme->rank; ++r) {
    int n = 0;
    for (int x = 0; x < 4; ++x) {
      const int c = scheme->a[r][x];
      if (c != 0 && c != 1 && c != -1) return 0;
      n += c != 0;
    }
    if (n < 1 || n > 2) return 0;
  }
  return 1;
}

extern "C" int lcg_gemm_r7_fused(const lcg_scheme_t* scheme, const void* a, int64_t lda,
                                 const void* b_planes, int64_t ld_b, void* c, int64_t ldc, int64_t M,
                                 int64_t N, int64_t K, int schedule, int cta_group, int32_t* status,
                                 void* stream) {
  if (!scheme || !a || !b_planes || !c) return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (schedule != LCG_SCHEDULE_ALL_RANKS && schedule != LCG_SCHEDULE_RANK_SPLIT &&
      schedule != LCG_SCHEDULE_HYBRID)
    return fail(LCG_ERR_BAD_ARG, "unknown schedule %d", schedule);
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  if (K < 128 || K % 128 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE,
                "the fused A producer reads whole 64-column K blocks of each half of A: K %% 128 must "
                "be 0, got K=%lld (use lcg_a_planes + lcg_gemm_r7)", (long long)K);
  R7Geometry g;
  if (int e = r7_geometry(M, N, K, &g)) return e;
  if (ldc < N) return fail(LCG_ERR_BAD_ARG, "ldc below N");
  if (lda < K || ld_b < g.k2p) return fail(LCG_ERR_BAD_ARG, "leading dimension below extent");
  CUtensorMap ma, mb;
  CMaps mc;
  GemmParams p;
  FuseParams fuse;
  if (int e = fill_fuse(scheme, a, lda, M, K, g, &fuse)) return e;      // the scheme, before any driver call
  if (int e = fill_r7(scheme, a, lda, b_planes, ld_b, c, ldc, M, N, g, schedule, cta_group, &ma, &mb,
                      &mc, &p, 0, -1, 0, K))
    return e;
  p.fuse = fuse;
  p.status = status;
  auto st_ = static_cast<cudaStream_t>(stream);
  if (int e = zero_tail_tiles(p, c, ldc, M, N, g, cta_group, st_)) return e;
  return cta_group == 1 ? launch<1, kModeFusedA>(ma, mb, mc, p, st_) : launch<2, kModeFusedA>(ma, mb, mc, p, st_);
}

// ---- product-ahead form: scratch layout = [256 bytes: chunk counters][planes of the two-term products]
constexpr int64_t kAheadHeaderBytes = 256;
constexpr int kAheadChunkRows = 4;

extern "C" int64_t lcg_gemm_r7_ahead_scratch_bytes(const lcg_scheme_t* scheme, int64_t M, int64_t K) {
  if (!scheme || M < 2 || K < 128 || K % 128 != 0) return -1;
  int slots = 0;
  for (int r = 0; r < scheme->rank; ++r) {
    int n = 0, neg = 0;
    for (int x = 0; x < 4; ++x) {
      n += scheme->a[r][x] != 0;
      neg |= scheme->a[r][x] < 0;
    }
    if (n < 1 || n > 2) return -1;
    if (!(n == 1 && !neg)) ++slots;
  }
  const int64_t m2 = (M + 1) / 2;
  return kAheadHeaderBytes + slots * m2 * (K / 2) * 2;
}

extern "C" int lcg_gemm_r7_ahead(const lcg_scheme_t* scheme, const void* a, int64_t lda,
                                 const void* b_planes, int64_t ld_b, void* c, int64_t ldc, int64_t M,
                                 int64_t N, int64_t K, void* scratch, int64_t scratch_bytes,
                                 int schedule, int cta_group, int32_t* status, void* stream) {
  if (!scheme || !a || !b_planes || !c || !scratch) return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (schedule != LCG_SCHEDULE_ALL_RANKS && schedule != LCG_SCHEDULE_RANK_SPLIT &&
      schedule != LCG_SCHEDULE_HYBRID)
    return fail(LCG_ERR_BAD_ARG, "unknown schedule %d", schedule);
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  if (K < 128 || K % 128 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE,
                "the in-kernel A planes cover whole 64-column K blocks of each half of A: K %% 128 must "
                "be 0, got K=%lld (use lcg_a_planes + lcg_gemm_r7)", (long long)K);
  if ((reinterpret_cast<uintptr_t>(a) & 15u) != 0 || lda % 8 != 0)
    return fail(LCG_ERR_MISALIGNED, "A must be 16-byte aligned with lda %% 8 == 0");
  if ((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0)
    return fail(LCG_ERR_MISALIGNED, "scratch must be 256-byte aligned");
  R7Geometry g;
  if (int e = r7_geometry(M, N, K, &g)) return e;
  if (ldc < N) return fail(LCG_ERR_BAD_ARG, "ldc below N");
  if (lda < K || ld_b < g.k2p) return fail(LCG_ERR_BAD_ARG, "leading dimension below extent");
  CUtensorMap ma, mb, ma2;
  CMaps mc;
  GemmParams p;
  FuseParams f;
  if (int e = fill_fuse(scheme, a, lda, M, K, g, &f)) return e;         // the scheme, before any driver call
  f.nslots = 0;
  for (int r = 0; r < scheme->rank; ++r) {
    f.slot[r] = -1;
    if (f.simt[r]) {
      f.slot[r] = static_cast<int8_t>(f.nslots);
      f.order[f.nslots++] = static_cast<int8_t>(r);
    }
  }
  const int64_t need = kAheadHeaderBytes + static_cast<int64_t>(f.nslots) * g.m2 * (K / 2) * 2;
  if (scratch_bytes < need)
    return fail(LCG_ERR_BAD_ARG, "scratch holds %lld bytes, this shape needs %lld "
                "(lcg_gemm_r7_ahead_scratch_bytes)", (long long)scratch_bytes, (long long)need);
  f.counters = static_cast<uint32_t*>(scratch);
  f.scratch = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(scratch) + kAheadHeaderBytes);
  f.chunk_rows = kAheadChunkRows;
  f.chunks = static_cast<int32_t>((g.m2 + kAheadChunkRows - 1) / kAheadChunkRows);
  if (int e = fill_r7(scheme, a, lda, b_planes, ld_b, c, ldc, M, N, g, schedule, cta_group, &ma, &mb,
                      &mc, &p, 0, -1, 0, K))
    return e;
  p.fuse = f;
  p.status = status;
  auto st_ = static_cast<cudaStream_t>(stream);
  if (f.nslots > 0) {
    if (int e = make_map(&ma2, f.scratch, K / 2, static_cast<int64_t>(f.nslots) * g.m2, K / 2, kBM,
                         "A plane scratch"))
      return e;
  } else {
    ma2 = ma;
  }
  LCG_CUDA_OK(cudaMemsetAsync(scratch, 0, kAheadHeaderBytes, st_));
  if (int e = zero_tail_tiles(p, c, ldc, M, N, g, cta_group, st_)) return e;
  return cta_group == 1 ? launch<1, kModeAheadA>(ma, mb, mc, p, st_, &ma2)
                        : launch<2, kModeAheadA>(ma, mb, mc, p, st_, &ma2);
}

extern "C" int lcg_gemm_r7_slab(const lcg_scheme_t* scheme, const void* a_planes, int64_t ld_a,
                                const void* b_planes, int64_t ld_b, void* c, int64_t ldc, int64_t M,
                                int64_t N, int64_t K, int schedule, int cta_group, int tile_row_begin,
                                int tile_row_end, int max_groups, int32_t* status, void* stream) {
  if (!scheme || !a_planes || !b_planes || !c) return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (schedule != LCG_SCHEDULE_ALL_RANKS && schedule != LCG_SCHEDULE_RANK_SPLIT &&
      schedule != LCG_SCHEDULE_HYBRID)
    return fail(LCG_ERR_BAD_ARG, "unknown schedule %d", schedule);
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  if (max_groups < 0) return fail(LCG_ERR_BAD_ARG, "max_groups must be >= 0");
  R7Geometry g;
  if (int e = r7_geometry(M, N, K, &g)) return e;
  if (ldc < N) return fail(LCG_ERR_BAD_ARG, "ldc below N");
  if (ld_a < g.k2p || ld_b < g.k2p) return fail(LCG_ERR_BAD_ARG, "plane leading dimension below K2p");
  CUtensorMap ma, mb;
  CMaps mc;
  GemmParams p;
  if (int e = fill_r7(scheme, a_planes, ld_a, b_planes, ld_b, c, ldc, M, N, g, schedule, cta_group,
                      &ma, &mb, &mc, &p, tile_row_begin, tile_row_end, max_groups))
    return e;
  p.status = status;
  auto st_ = static_cast<cudaStream_t>(stream);
  if (int e = zero_tail_tiles(p, c, ldc, M, N, g, cta_group, st_)) return e;
  return cta_group == 1 ? launch<1, kModePlain>(ma, mb, mc, p, st_) : launch<2, kModePlain>(ma, mb, mc, p, st_);
}

static int gate_up_chain(const lcg_scheme_t* scheme, const lcg_scheme_t* plane_scheme,
                         const void* a_planes, int64_t ld_a, const void* b_planes, int64_t ld_b,
                         void* z, int64_t ldz, int64_t M, int64_t N, int64_t K, void* down_planes,
                         int64_t ld_planes, void* preclear, int64_t preclear_bytes,
                         const void* preload, int schedule, int cta_group, int32_t* status,
                         void* stream) {
  if (!scheme || !plane_scheme || !a_planes || !b_planes || !z || !down_planes)
    return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (preload != nullptr) {
    if (preclear == nullptr || preclear_bytes <= 0)
      return fail(LCG_ERR_BAD_ARG, "an initial content needs the consumer output it is written to");
    if ((reinterpret_cast<uintptr_t>(preload) & 15u) != 0)
      return fail(LCG_ERR_MISALIGNED, "the initial content must be 16-byte aligned");
    const auto a0 = reinterpret_cast<uintptr_t>(preload), b0 = reinterpret_cast<uintptr_t>(preclear);
    if (a0 < b0 + static_cast<uintptr_t>(preclear_bytes) && b0 < a0 + static_cast<uintptr_t>(preclear_bytes))
      return fail(LCG_ERR_BAD_ARG, "the initial content overlaps the consumer output");
  }
  if (schedule != LCG_SCHEDULE_ALL_RANKS && schedule != LCG_SCHEDULE_HYBRID)
    return fail(LCG_ERR_BAD_ARG, "the chained GEMM runs the all-ranks or the hybrid schedule, got %d",
                schedule);
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  if (M % 2 != 0 || N % 256 != 0 || K % 128 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE,
                "chained gate_up needs an even M, N %% 256 == 0 (I %% 128 == 0) and K %% 128 == 0; "
                "got M=%lld N=%lld K=%lld",
                (long long)M, (long long)N, (long long)K);
  R7Geometry g;
  if (int e = r7_geometry(M, N, K, &g)) return e;
  const int64_t inter = N / 2;
  if (g.n2 != inter) return fail(LCG_ERR_UNSUPPORTED_SHAPE, "gate/up split does not fall on a block");
  if (ldz < N || ld_planes < inter / 2 || ld_planes % 8 != 0)
    return fail(LCG_ERR_BAD_ARG, "bad leading dimensions");
  if (ld_a < g.k2p || ld_b < g.k2p) return fail(LCG_ERR_BAD_ARG, "plane leading dimension below K2p");
  if ((reinterpret_cast<uintptr_t>(down_planes) & 15u) != 0)
    return fail(LCG_ERR_MISALIGNED, "down planes must be 16-byte aligned");
  if (preclear != nullptr &&
      (preclear_bytes < 0 || preclear_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(preclear) & 15u) != 0))
    return fail(LCG_ERR_MISALIGNED, "preclear region must be 16-byte aligned and sized");
  CUtensorMap ma, mb;
  CMaps mc;
  GemmParams p;
  if (int e = fill_r7(scheme, a_planes, ld_a, b_planes, ld_b, z, ldz, M, N, g, schedule, cta_group,
                      &ma, &mb, &mc, &p))
    return e;
  p.status = status;
  ChainParams& ch = p.chain;
  ch.z = static_cast<const __nv_bfloat16*>(z);
  ch.ldz = ldz;
  ch.planes = static_cast<__nv_bfloat16*>(down_planes);
  ch.ld_planes = ld_planes;
  ch.m2 = static_cast<int32_t>(g.m2);
  ch.inter = static_cast<int32_t>(inter);
  ch.plane_rank = plane_scheme->rank;
  for (int r = 0; r < plane_scheme->rank; ++r)
    for (int x = 0; x < 4; ++x) ch.plane_terms.coef[r][x] = static_cast<float>(plane_scheme->a[r][x]);
  ch.preclear = preclear_bytes > 0 ? static_cast<uint4*>(preclear) : nullptr;
  ch.preclear_vecs = preclear_bytes / 16;
  ch.preload = ch.preclear != nullptr ? static_cast<const uint4*>(preload) : nullptr;
  auto st_ = static_cast<cudaStream_t>(stream);
  if (int e = zero_tail_tiles(p, z, ldz, M, N, g, cta_group, st_)) return e;
  // The plane phase is compiled for the shipped `down` scheme's A table; any other table runs
  // the same kernel with the table read at run time.
  const bool fixed = table_code(ch.plane_terms, plane_scheme->rank) == kCodeLocalityA;
  int e = LCG_OK;
  if (cta_group == 1)
    e = fixed ? launch<1, kModePlanes, kCodeLocalityA>(ma, mb, mc, p, st_) : launch<1, kModePlanes>(ma, mb, mc, p, st_);
  else
    e = fixed ? launch<2, kModePlanes, kCodeLocalityA>(ma, mb, mc, p, st_) : launch<2, kModePlanes>(ma, mb, mc, p, st_);
  if (e) return e;
  if (p.tail_tiles > 0) {
    const int tile_m = kBM * cta_group;
    const unsigned tail_grid = static_cast<unsigned>(p.tail_tiles * (tile_m / 32));
    if (fixed)
      k_tail_planes<kCodeLocalityA><<<tail_grid, kPlaneThreads, 0, st_>>>(p, tile_m);
    else
      k_tail_planes<0><<<tail_grid, kPlaneThreads, 0, st_>>>(p, tile_m);
    LCG_CUDA_OK(cudaGetLastError());
    count_launch();
  }
  return LCG_OK;
}

extern "C" int lcg_gate_up_chain(const lcg_scheme_t* scheme, const lcg_scheme_t* plane_scheme,
                                 const void* a_planes, int64_t ld_a, const void* b_planes,
                                 int64_t ld_b, void* z, int64_t ldz, int64_t M, int64_t N, int64_t K,
                                 void* down_planes, int64_t ld_planes, void* preclear,
                                 int64_t preclear_bytes, int schedule, int cta_group,
                                 int32_t* status, void* stream) {
  return gate_up_chain(scheme, plane_scheme, a_planes, ld_a, b_planes, ld_b, z, ldz, M, N, K, down_planes,
                       ld_planes, preclear, preclear_bytes, nullptr, schedule, cta_group, status, stream);
}

extern "C" int lcg_gate_up_chain_init(const lcg_scheme_t* scheme, const lcg_scheme_t* plane_scheme,
                                      const void* a_planes, int64_t ld_a, const void* b_planes,
                                      int64_t ld_b, void* z, int64_t ldz, int64_t M, int64_t N,
                                      int64_t K, void* down_planes, int64_t ld_planes, void* consumer_out,
                                      int64_t consumer_bytes, const void* init_from, int schedule,
                                      int cta_group, int32_t* status, void* stream) {
  if (!init_from) return fail(LCG_ERR_BAD_ARG, "NULL initial content");
  return gate_up_chain(scheme, plane_scheme, a_planes, ld_a, b_planes, ld_b, z, ldz, M, N, K, down_planes,
                       ld_planes, consumer_out, consumer_bytes, init_from, schedule, cta_group, status,
                       stream);
}

extern "C" int lcg_gemm_r7_push(const lcg_scheme_t* scheme, const void* a_planes, int64_t ld_a,
                                const void* b_planes, int64_t ld_b, void* c, int64_t ldc, int64_t M,
                                int64_t N, int64_t K, void* const* slots, int world, int rank,
                                int64_t rows_per_owner, int cta_group, int32_t* status,
                                void* stream) {
  if (!scheme || !a_planes || !b_planes || !c || !slots) return fail(LCG_ERR_BAD_ARG, "NULL operand");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return fail(LCG_ERR_BAD_ARG, "world must be 1..%d and rank inside it; got world=%d rank=%d",
                kMaxWorld, world, rank);
  if (rows_per_owner < 1 || rows_per_owner * world < M)
    return fail(LCG_ERR_BAD_ARG, "rows_per_owner * world must cover M");
  if (N % 8 != 0) return fail(LCG_ERR_UNSUPPORTED_SHAPE, "the push moves 16-byte vectors: N %% 8 must be 0");
  for (int w = 0; w < world; ++w) {
    if (!slots[w]) return fail(LCG_ERR_BAD_ARG, "NULL slot pointer for owner %d", w);
    if ((reinterpret_cast<uintptr_t>(slots[w]) & 15u) != 0)
      return fail(LCG_ERR_MISALIGNED, "slot pointers must be 16-byte aligned");
  }
  cta_group = resolve_group(cta_group);
  if (cta_group != 1 && cta_group != 2) return fail(LCG_ERR_BAD_ARG, "cta_group must be 0, 1 or 2");
  R7Geometry g;
  if (int e = r7_geometry(M, N, K, &g)) return e;
  if (ldc < N || ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(c) & 15u) != 0)
    return fail(LCG_ERR_MISALIGNED, "C must be 16-byte aligned with ldc %% 8 == 0 and ldc >= N");
  if (ld_a < g.k2p || ld_b < g.k2p) return fail(LCG_ERR_BAD_ARG, "plane leading dimension below K2p");
  CUtensorMap ma, mb;
  CMaps mc;
  GemmParams p;
  if (int e = fill_r7(scheme, a_planes, ld_a, b_planes, ld_b, c, ldc, M, N, g, LCG_SCHEDULE_HYBRID,
                      cta_group, &ma, &mb, &mc, &p))
    return e;
  p.status = status;
  PushParams& pp = p.push;
  pp.c = static_cast<const __nv_bfloat16*>(c);
  pp.ldc = ldc;
  for (int w = 0; w < world; ++w) pp.slot[w] = static_cast<__nv_bfloat16*>(slots[w]);
  pp.world = world;
  pp.rows_per_owner = static_cast<int32_t>(rows_per_owner);
  pp.m = static_cast<int32_t>(M);
  pp.n = static_cast<int32_t>(N);
  pp.m2 = static_cast<int32_t>(g.m2);
  pp.n2 = static_cast<int32_t>(g.n2);
  // Every rank walks the tile rows in the same order, and a tile row's rows belong to two owners: left
  // alone, all ranks push to the same two owners at any moment and those two inbound links carry the
  // whole exchange while the others idle.  Rank r therefore starts its walk r / world of the way down.
  p.tm_rot = static_cast<int32_t>((static_cast<int64_t>(rank) * p.tiles_m) / world);
  auto st_ = static_cast<cudaStream_t>(stream);
  if (int e = zero_tail_tiles(p, c, ldc, M, N, g, cta_group, st_)) return e;
  if (int e = cta_group == 1 ? launch<1, kModePush>(ma, mb, mc, p, st_) : launch<2, kModePush>(ma, mb, mc, p, st_))
    return e;
  if (p.tail_tiles > 0) {
    const int tile_m = kBM * cta_group;
    k_tail_planes<0><<<p.tail_tiles * (tile_m / 32), kPlaneThreads, 0, st_>>>(p, tile_m);
    LCG_CUDA_OK(cudaGetLastError());
    count_launch();
  }
  return LCG_OK;
}

extern "C" int lcg_describe_gemm(int64_t M, int64_t N, int64_t K, int rank7, int schedule,
                                 int cta_group, char* buf, int buflen) {
  if (buf == nullptr || buflen < 1) return fail(LCG_ERR_BAD_ARG, "no buffer");
  cta_group = resolve_group(cta_group);
  const int tile_m = kBM * cta_group;
  const int stages = cta_group == 1 ? Tile<1>::kStages : Tile<2>::kStages;
  const int smem = cta_group == 1 ? Tile<1>::kSmemBytes : Tile<2>::kSmemBytes;
  int64_t rows = M, cols = N, kk = K;
  if (rank7) {
    R7Geometry g;
    if (int e = r7_geometry(M, N, K, &g)) return e;
    rows = g.m2;
    cols = g.n2;
    kk = g.k2p;
  }
  const int64_t tm = (rows + tile_m - 1) / tile_m, tn = (cols + kBN - 1) / kBN;
  const int groups = sm_count() / cta_group;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.num_units = static_cast<int>(tm * tn);
  if (rank7) plan_units(7, static_cast<int>(tm * tn), groups, static_cast<int>((kk + kBK - 1) / kBK), schedule, &p);
  const int64_t units = p.num_units;
  return snprintf(buf, buflen,
                  "%s %lldx%lldx%lld: tile %dx%dx%d cta_group=%d stages=%d smem=%dB tmem=512 cols (2 acc "
                  "stages); %lldx%lld tiles, %lld units over %d CTA groups (%.2f waves), %lld k-blocks/step",
                  rank7 ? (schedule == LCG_SCHEDULE_RANK_SPLIT ? "rank7/rank-split"
                           : schedule == LCG_SCHEDULE_HYBRID ? "rank7/hybrid" : "rank7/all-ranks")
                        : "dense",
                  (long long)M, (long long)K, (long long)N, tile_m, kBN, kBK, cta_group, stages, smem,
                  (long long)tm, (long long)tn, (long long)units, groups,
                  static_cast<double>(units) / groups, (long long)((kk + kBK - 1) / kBK));
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded-wait machinery: one CTA waits on an mbarrier that nothing ever
// arrives at, with a short limit.  The wait must run out, record `kCodeSelfTest` in the status
// word and let the kernel return normally; the context stays usable.
namespace lcg {
constexpr int kCodeSelfTest = 199;
__global__ void k_selftest_wait(int32_t* status, uint64_t limit_ns, int* finished) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0u;
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtl ctl{&abort_flag, status, limit_ns};
  mbar_wait(smem_u32(&bar), 0u, ctl, kCodeSelfTest);     // phase 0 never completes
  mbar_wait(smem_u32(&bar), 0u, ctl, kCodeSelfTest);     // a later wait returns at once
  __syncthreads();
  if (threadIdx.x == 0 && finished != nullptr) *finished = abort_flag != 0u ? 1 : 0;
}
}  // namespace lcg

extern "C" int lcg_selftest_wait_timeout(int32_t* status, int64_t limit_us, int32_t* finished,
                                         void* stream) {
  if (status == nullptr) return fail(LCG_ERR_BAD_ARG, "status must not be NULL");
  if (limit_us < 1 || limit_us > 1000000) return fail(LCG_ERR_BAD_ARG, "limit_us outside [1, 1e6]");
  k_selftest_wait<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      status, static_cast<uint64_t>(limit_us) * 1000ull, finished);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}
