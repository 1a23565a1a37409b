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
