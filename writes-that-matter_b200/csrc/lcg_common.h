// Shared host-side declarations: error reporting, the scheme handle and the
// per-step tables the GEMM kernel receives as launch parameters.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lcgemm_b200.h"

namespace lcg {

constexpr int kMaxRank = 7;

// ---- error reporting (thread-local text behind lcg_last_error) -----------
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);

#define LCG_CUDA_OK(expr)                                                        \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess)                                                       \
      return ::lcg::fail(LCG_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// ---- what the kernel needs to know about one accumulator step -------------
struct EpiDest {
  int8_t bi, bj;     // destination C block
  int8_t first;      // 1: plain store (initialises the block), 0: reduce-add
  int8_t pad;
};
struct EpiGroup {      // one TMEM->smem staging pass and the blocks it feeds
  int32_t coeff;       // +1 / -1 (any small integer)
  int32_t ndest;
  EpiDest dest[4];
};
struct StepDesc {
  int32_t a_plane;     // which A plane / B plane the product reads
  int32_t b_plane;
  int32_t clear;       // 1: first MMA overwrites the accumulator
  int32_t ngroups;
  EpiGroup group[2];
};

// Signed-sum tables for the SIMT plane producers: per rank, coefficient of
// each of the four blocks (row-major over the 2x2 block grid).
// Stored as floats: an int-to-float conversion per use would go through the SM's quarter-rate
// conversion pipe, which is what these HBM-bound kernels run out of first.
struct TermTable {
  float coef[kMaxRank][4];
};

// A coefficient table whose entries are all -1, 0 or +1, packed two bits per entry (entry
// r * 4 + x at bit 2 * (r * 4 + x): 0 = zero, 1 = +1, 3 = -1).  Kernels templated on the packed
// code see the table at compile time: the signed sums become straight adds and subtracts with
// no table loads, compares or branches (these kernels are bound by instruction issue).
__host__ __device__ constexpr int code_coef(unsigned long long code, int r, int x) {
  return static_cast<int>((code >> (2 * (r * 4 + x))) & 3ull);
}
constexpr unsigned long long pack_code(const int (&t)[kMaxRank][4]) {
  unsigned long long code = 0;
  for (int r = 0; r < kMaxRank; ++r)
    for (int x = 0; x < 4; ++x)
      code |= static_cast<unsigned long long>(t[r][x] == 0 ? 0 : (t[r][x] > 0 ? 1 : 3)) << (2 * (r * 4 + x));
  return code;
}
// The A-side tables of the two schemes this package ships (lcgemm/schemes/*.json).
constexpr int kTablePostsumA[kMaxRank][4] = {{0, 1, 0, 0},  {1, 0, 0, 0}, {0, 1, 1, -1}, {0, 1, 0, -1},
                                             {0, 0, 1, -1}, {0, 0, 1, 0}, {1, -1, -1, 1}};
constexpr int kTableLocalityA[kMaxRank][4] = {{-1, 0, 1, 0}, {0, 0, 1, 1}, {0, 0, 0, 1}, {1, 0, 0, 1},
                                              {1, 0, 0, 0},  {1, 1, 0, 0}, {0, 1, 0, -1}};
constexpr unsigned long long kCodePostsumA = pack_code(kTablePostsumA);
constexpr unsigned long long kCodeLocalityA = pack_code(kTableLocalityA);

// 0 when the table is not all -1 / 0 / +1 or not of full rank; else its packed code.
inline unsigned long long table_code(const TermTable& t, int rank) {
  if (rank != kMaxRank) return 0;
  unsigned long long code = 0;
  for (int r = 0; r < kMaxRank; ++r)
    for (int x = 0; x < 4; ++x) {
      const float v = t.coef[r][x];
      if (v != 0.f && v != 1.f && v != -1.f) return 0;
      code |= static_cast<unsigned long long>(v == 0.f ? 0 : (v > 0.f ? 1 : 3)) << (2 * (r * 4 + x));
    }
  return code;
}

}  // namespace lcg

// The opaque handle of the C ABI.
struct lcg_scheme {
  int rank;
  int has_postsum;
  int8_t a[lcg::kMaxRank][4];
  int8_t b[lcg::kMaxRank][4];
  int8_t c[lcg::kMaxRank][4];
  int8_t clear[lcg::kMaxRank];       // acc_clear: all ones without a plan
  lcg::StepDesc all_ranks[lcg::kMaxRank];   // epi_groups walk, store-first
  lcg::StepDesc rank_split[lcg::kMaxRank];  // every product alone, reduce-add only
};
