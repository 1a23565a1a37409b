// HBM-bound SIMT kernels of the path: operand-plane producers (weights offline,
// activations per call), the fused residual + RMSNorm + A-plane seam, the
// SwiGLU + A-plane seam as a kernel of its own, and the stock layer's seams for
// the dense arm.  All of them move 16-byte vectors (8 bf16), do their
// arithmetic in fp32 and round once on the way out.
#include <cuda_bf16.h>

#include "lcg_common.h"

namespace lcg {
namespace {

struct alignas(16) Vec8 {
  __nv_bfloat162 v[4];
};

// bf16 -> fp32 is a 16-bit shift: done with integer ops so that it stays off the conversion pipe.
__device__ __forceinline__ void unpack8(const Vec8& p, float (&f)[8]) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&p.v[t]);
    f[2 * t] = __uint_as_float(w << 16);
    f[2 * t + 1] = __uint_as_float(w & 0xffff0000u);
  }
}

__device__ __forceinline__ Vec8 pack8(const float (&f)[8]) {
  Vec8 p;
#pragma unroll
  for (int t = 0; t < 4; ++t) p.v[t] = __floats2bfloat162_rn(f[2 * t], f[2 * t + 1]);
  return p;
}

__device__ __forceinline__ Vec8 zero8() {
  Vec8 p;
#pragma unroll
  for (int t = 0; t < 4; ++t) p.v[t] = __floats2bfloat162_rn(0.f, 0.f);
  return p;
}

// Eight consecutive elements of row `row` starting at column `col` of a
// (rows, cols) matrix with leading dimension ld; anything outside is zero.
// `vec_ok` says 16-byte loads are legal for this matrix.
__device__ __forceinline__ void load8_guarded(const __nv_bfloat16* __restrict__ base, int64_t ld,
                                              int64_t rows, int64_t cols, int64_t row, int64_t col,
                                              int64_t col_limit, bool vec_ok, float (&f)[8]) {
  // col_limit: first column (exclusive bound) this block may read, <= cols.
  if (row >= rows || col >= col_limit) {
#pragma unroll
    for (int t = 0; t < 8; ++t) f[t] = 0.f;
    return;
  }
  const __nv_bfloat16* p = base + row * ld + col;
  if (vec_ok && col + 8 <= col_limit) {
    unpack8(*reinterpret_cast<const Vec8*>(p), f);
    return;
  }
#pragma unroll
  for (int t = 0; t < 8; ++t)
    f[t] = (col + t < col_limit)
               ? __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(p + t)) << 16)
               : 0.f;
}

__device__ __forceinline__ void signed_sum(const TermTable& tt, int r, const float (&blk)[4][8],
                                           float (&out)[8]) {
  // Starts from +0 and adds term by term in block order, so a sum of zeros is +0 whatever
  // the signs of the coefficients (a bare -1 * 0 would be -0).
#pragma unroll
  for (int t = 0; t < 8; ++t) out[t] = 0.f;
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const float w = tt.coef[r][x];
    if (w == 0.f) continue;
#pragma unroll
    for (int t = 0; t < 8; ++t) out[t] = fmaf(w, blk[x][t], out[t]);
  }
}

// Same result as signed_sum (starts from +0, block order), table known at compile time.
template <unsigned long long kCode>
__device__ __forceinline__ void signed_sum_fixed(int r, const float (&blk)[4][8], float (&out)[8]) {
#pragma unroll
  for (int t = 0; t < 8; ++t) out[t] = 0.f;
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const int c = code_coef(kCode, r, x);      // a constant once the caller's loop over r is unrolled
    if (c == 1) {
#pragma unroll
      for (int t = 0; t < 8; ++t) out[t] = __fadd_rn(out[t], blk[x][t]);   // never contracted
    } else if (c == 3) {
#pragma unroll
      for (int t = 0; t < 8; ++t) out[t] = __fsub_rn(out[t], blk[x][t]);
    }
  }
}

// ------------------------------------------------------------------ planes
// One thread per (block row, 8-column vector).  `transposed_blocks` selects the
// block indexing: A planes combine src[i*R2 + row, k*K2 + col] with table index
// i*2 + k; B planes combine src[j*R2 + row, k*K2 + col] with table index k*2 + j.
template <unsigned long long kCode>      // 0: the table comes at run time in `tt`
__global__ void __launch_bounds__(128)
k_planes(const __nv_bfloat16* __restrict__ src, int64_t rows, int64_t cols, int64_t ld,
         int64_t rows2, int64_t k2, int64_t k2p, int rank, TermTable tt, bool b_side,
         bool vec_ok, __nv_bfloat16* __restrict__ out, int64_t ld_out) {
  const int64_t row = blockIdx.x;
  const int64_t v = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
  if (v * 8 >= k2p) return;
  const int64_t col = v * 8;
  float blk[4][8];
#pragma unroll
  for (int rb = 0; rb < 2; ++rb)
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      const int x = b_side ? kb * 2 + rb : rb * 2 + kb;
      const int64_t c0 = kb * k2 + col;
      const int64_t lim = min(cols, (kb + 1) * k2);
      // a column past this block's K2 is zero even when the matrix continues
      load8_guarded(src, ld, rows, cols, rb * rows2 + row, c0, (col < k2) ? lim : 0, vec_ok, blk[x]);
    }
  if constexpr (kCode != 0) {
#pragma unroll
    for (int r = 0; r < kMaxRank; ++r) {
      float o[8];
      signed_sum_fixed<kCode>(r, blk, o);
      *reinterpret_cast<Vec8*>(out + (r * rows2 + row) * ld_out + col) = pack8(o);
    }
  } else {
    for (int r = 0; r < rank; ++r) {
      float o[8];
      signed_sum(tt, r, blk, o);
      *reinterpret_cast<Vec8*>(out + (r * rows2 + row) * ld_out + col) = pack8(o);
    }
  }
}

// ------------------------------------------------- residual + RMSNorm + planes
template <int VPT>
__global__ void __launch_bounds__(1024)
k_norm_planes(const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ residual,
              const __nv_bfloat16* __restrict__ norm_w, int64_t m2, int64_t k, int64_t k2p,
              float eps, int rank, TermTable tt, __nv_bfloat16* residual_out,
              __nv_bfloat16* __restrict__ out, int64_t ld_out) {
  // One CTA per row pair (rho, rho + M/2): both rows feed every plane row rho.
  __shared__ float s_part[2][32];
  const int64_t rho = blockIdx.x;
  const int64_t k2 = k / 2;
  const int64_t nvec = k2 / 8;
  const int64_t nvec_p = k2p / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;

  Vec8 h[VPT][2][2];
  float ss[2] = {0.f, 0.f};
#pragma unroll
  for (int t = 0; t < VPT; ++t) {
    const int64_t v = tid + static_cast<int64_t>(t) * blockDim.x;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        if (v < nvec) {
          const int64_t off = (i * m2 + rho) * k + kb * k2 + v * 8;
          if (delta != nullptr) {
            float d[8], r[8], s[8];
            unpack8(*reinterpret_cast<const Vec8*>(delta + off), d);
            unpack8(*reinterpret_cast<const Vec8*>(residual + off), r);
#pragma unroll
            for (int e = 0; e < 8; ++e) s[e] = d[e] + r[e];
            // The norm must see exactly the value that is stored as the new
            // residual stream, so round first.
            h[t][i][kb] = pack8(s);
          } else {
            h[t][i][kb] = *reinterpret_cast<const Vec8*>(residual + off);   // no delta: h is the residual
          }
          if (residual_out != nullptr) *reinterpret_cast<Vec8*>(residual_out + off) = h[t][i][kb];
          float hf[8];
          unpack8(h[t][i][kb], hf);
#pragma unroll
          for (int e = 0; e < 8; ++e) ss[i] = fmaf(hf[e], hf[e], ss[i]);
        } else {
          h[t][i][kb] = zero8();
        }
      }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    if (lane == 0) s_part[i][warp] = ss[i];
  }
  __syncthreads();
  float rstd[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float part = lane < nwarps ? s_part[i][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    rstd[i] = rsqrtf(part / static_cast<float>(k) + eps);
  }

#pragma unroll
  for (int t = 0; t < VPT; ++t) {
    const int64_t v = tid + static_cast<int64_t>(t) * blockDim.x;
    if (v >= nvec_p) continue;
    float y[4][8];
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      float w[8];
      if (v < nvec) {
        unpack8(*reinterpret_cast<const Vec8*>(norm_w + kb * k2 + v * 8), w);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float hf[8];
        unpack8(h[t][i][kb], hf);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[i * 2 + kb][e] = hf[e] * rstd[i] * (w[e] + 1.0f);
      }
    }
    for (int r = 0; r < rank; ++r) {
      float o[8];
      signed_sum(tt, r, y, o);
      *reinterpret_cast<Vec8*>(out + (r * m2 + rho) * ld_out + v * 8) = pack8(o);
    }
  }
}

// The same seam with the row pair staged in shared memory by cp.async: the loads of a CTA are
// in flight without holding registers, more CTAs fit per SM, and the rounded sum h overwrites the
// delta slot so that the second phase reads it back from shared memory.  Each thread only ever
// touches the vectors it copied itself.  Used when the four rows (2 rows x delta, residual) fit:
// 8 * K bytes of dynamic shared memory.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

template <unsigned long long kCode>      // 0: the table comes at run time in `tt`
__global__ void __launch_bounds__(512, 2)  // 64 registers: three 320-thread CTAs fit an SM
k_norm_planes_staged(const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ residual,
                     const __nv_bfloat16* __restrict__ norm_w, int m2, int k, float eps, int rank,
                     TermTable tt, __nv_bfloat16* residual_out, __nv_bfloat16* __restrict__ out,
                     int ld_out) {
  extern __shared__ __align__(16) unsigned char stage_raw[];
  __shared__ float s_part[2][16];
  Vec8* stage = reinterpret_cast<Vec8*>(stage_raw);      // [(i * 2 + kb) * 2 + operand][nvec]
  const int rho = blockIdx.x;
  const int k2 = k / 2;
  const int nvec = k2 / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;

  for (int v = tid; v < nvec; v += blockDim.x)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        const size_t off = (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8;
        if (delta != nullptr) cp_async16(&stage[((i * 2 + kb) * 2 + 0) * nvec + v], delta + off);
        cp_async16(&stage[((i * 2 + kb) * 2 + 1) * nvec + v], residual + off);
      }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  float ss[2] = {0.f, 0.f};
  for (int v = tid; v < nvec; v += blockDim.x)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        Vec8 h = stage[((i * 2 + kb) * 2 + 1) * nvec + v];      // no delta: h is the residual
        if (delta != nullptr) {
          float d[8], r[8], s[8];
          unpack8(stage[((i * 2 + kb) * 2 + 0) * nvec + v], d);
          unpack8(h, r);
#pragma unroll
          for (int e = 0; e < 8; ++e) s[e] = d[e] + r[e];
          h = pack8(s);                   // the norm sees exactly what is stored as the residual
        }
        const size_t off = (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8;
        if (residual_out != nullptr) *reinterpret_cast<Vec8*>(residual_out + off) = h;
        stage[((i * 2 + kb) * 2 + 0) * nvec + v] = h;
        float hf[8];
        unpack8(h, hf);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss[i] = fmaf(hf[e], hf[e], ss[i]);
      }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    if (lane == 0) s_part[i][warp] = ss[i];
  }
  __syncthreads();
  float rstd[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float part = lane < nwarps ? s_part[i][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    rstd[i] = rsqrtf(part / static_cast<float>(k) + eps);
  }

  for (int v = tid; v < nvec; v += blockDim.x) {
    float y[4][8];
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      float w[8];
      unpack8(*reinterpret_cast<const Vec8*>(norm_w + kb * k2 + v * 8), w);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float hf[8];
        unpack8(stage[((i * 2 + kb) * 2 + 0) * nvec + v], hf);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[i * 2 + kb][e] = hf[e] * rstd[i] * (w[e] + 1.0f);
      }
    }
    if constexpr (kCode != 0) {
      __nv_bfloat16* dst = out + static_cast<size_t>(rho) * ld_out + v * 8;
      const size_t plane_stride = static_cast<size_t>(m2) * ld_out;
#pragma unroll
      for (int r = 0; r < kMaxRank; ++r) {
        float o[8];
        signed_sum_fixed<kCode>(r, y, o);
        *reinterpret_cast<Vec8*>(dst + r * plane_stride) = pack8(o);
      }
    } else {
      for (int r = 0; r < rank; ++r) {
        float o[8];
        signed_sum(tt, r, y, o);
        *reinterpret_cast<Vec8*>(out + (static_cast<size_t>(r) * m2 + rho) * ld_out + v * 8) = pack8(o);
      }
    }
  }
}

// The same seam with everything in registers, for rows of at most 416 vectors per block column
// (K <= 6656): one thread owns vector v of all four blocks of the row pair.  All eight loads of a
// thread are issued before anything is consumed (they are its whole share of the memory-level
// parallelism), the rounded sum h stays in registers as bf16, and the residual stream is stored
// before the barrier so that it streams out while the CTA waits there
// (lcgemm/kernels/fused_norm.py:166-198).  Two CTAs to an SM.
__device__ __forceinline__ Vec8 ldg_stream(const __nv_bfloat16* p) {
  const uint4 q = __ldcs(reinterpret_cast<const uint4*>(p));
  return *reinterpret_cast<const Vec8*>(&q);
}
__device__ __forceinline__ void stg_stream(__nv_bfloat16* p, const Vec8& v) {
  __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&v));
}

template <unsigned long long kCode>      // the packed A table (compile time only)
__global__ void __launch_bounds__(416, 2)
k_norm_planes_reg(const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ residual,
                  const __nv_bfloat16* __restrict__ norm_w, int m2, int k, float eps,
                  __nv_bfloat16* residual_out, __nv_bfloat16* __restrict__ out, int ld_out) {
  __shared__ float s_part[2][16];
  const int rho = blockIdx.x;
  const int k2 = k / 2;
  const int nvec = k2 / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const bool live = tid < nvec;
  const int v = live ? tid : 0;

  Vec8 d[2][2], r[2][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      const size_t off = (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8;
      d[i][kb] = ldg_stream(delta + off);
      r[i][kb] = ldg_stream(residual + off);
    }
  float w[2][8];
#pragma unroll
  for (int kb = 0; kb < 2; ++kb) {
    unpack8(*reinterpret_cast<const Vec8*>(norm_w + kb * k2 + v * 8), w[kb]);
#pragma unroll
    for (int e = 0; e < 8; ++e) w[kb][e] += 1.0f;
  }
  Vec8 h[2][2];
  float ss[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      float df[8], rf[8], sf[8];
      unpack8(d[i][kb], df);
      unpack8(r[i][kb], rf);
#pragma unroll
      for (int e = 0; e < 8; ++e) sf[e] = df[e] + rf[e];
      h[i][kb] = pack8(sf);               // the norm sees exactly what is stored as the residual
      if (live)
        stg_stream(residual_out + (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8, h[i][kb]);
      float hf[8];
      unpack8(h[i][kb], hf);
      if (live) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ss[i] = fmaf(hf[e], hf[e], ss[i]);
      }
    }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    if (lane == 0) s_part[i][warp] = ss[i];
  }
  __syncthreads();
  float rstd[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float part = lane < nwarps ? s_part[i][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    rstd[i] = rsqrtf(part / static_cast<float>(k) + eps);
  }
  if (!live) return;
  float y[4][8];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      float hf[8];
      unpack8(h[i][kb], hf);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[i * 2 + kb][e] = hf[e] * rstd[i] * w[kb][e];
    }
  __nv_bfloat16* dst = out + static_cast<size_t>(rho) * ld_out + v * 8;
  const size_t plane_stride = static_cast<size_t>(m2) * ld_out;
#pragma unroll
  for (int rr = 0; rr < kMaxRank; ++rr) {
    float o[8];
    signed_sum_fixed<kCode>(rr, y, o);
    stg_stream(dst + rr * plane_stride, pack8(o));
  }
}

// The register form at 64 registers, for rows of up to 512 vectors per block column (K <= 8192)
// and for a call without a delta.  Two 512-thread CTAs fit an SM because nothing but h (packed
// bf16) lives across the barrier: each plane recomputes its normalised terms from h, the row's
// 1 / rms and the weight vector -- the same multiplications in the same order as the other forms,
// so the same bits.  kHasDelta false: h is the residual itself, no sum is formed and nothing is
// stored for the residual stream (four loads and seven stores per thread instead of eight and
// eleven).
template <unsigned long long kCode, bool kHasDelta>
__global__ void __launch_bounds__(512, 2)
k_norm_planes_lean(const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ norm_w, int m2, int k, float eps,
                   __nv_bfloat16* residual_out, __nv_bfloat16* __restrict__ out, int ld_out) {
  __shared__ float s_part[2][16];
  const int rho = blockIdx.x;
  const int k2 = k / 2;
  const int nvec = k2 / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const bool live = tid < nvec;
  const int v = live ? tid : 0;

  Vec8 h[2][2];
  if constexpr (kHasDelta) {
    Vec8 d[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        const size_t off = (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8;
        d[i][kb] = ldg_stream(delta + off);
        h[i][kb] = ldg_stream(residual + off);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        float df[8], rf[8], sf[8];
        unpack8(d[i][kb], df);
        unpack8(h[i][kb], rf);
#pragma unroll
        for (int e = 0; e < 8; ++e) sf[e] = df[e] + rf[e];
        h[i][kb] = pack8(sf);             // the norm sees exactly what is stored as the residual
        if (live && residual_out != nullptr)
          stg_stream(residual_out + (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8, h[i][kb]);
      }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
        h[i][kb] = ldg_stream(residual + (static_cast<size_t>(i) * m2 + rho) * k + kb * k2 + v * 8);
  }
  float ss[2] = {0.f, 0.f};
  if (live) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        float hf[8];
        unpack8(h[i][kb], hf);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss[i] = fmaf(hf[e], hf[e], ss[i]);
      }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    if (lane == 0) s_part[i][warp] = ss[i];
  }
  __syncthreads();
  float rstd[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float part = lane < nwarps ? s_part[i][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    rstd[i] = rsqrtf(part / static_cast<float>(k) + eps);
  }
  if (!live) return;
  Vec8 wv[2];
#pragma unroll
  for (int kb = 0; kb < 2; ++kb) wv[kb] = *reinterpret_cast<const Vec8*>(norm_w + kb * k2 + v * 8);
  __nv_bfloat16* dst = out + static_cast<size_t>(rho) * ld_out + v * 8;
  const size_t plane_stride = static_cast<size_t>(m2) * ld_out;
#pragma unroll
  for (int rr = 0; rr < kMaxRank; ++rr) {
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = 0.f;          // from +0, block order, as signed_sum_fixed
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int c = code_coef(kCode, rr, x);
      if (c != 1 && c != 3) continue;
      float hf[8], wf[8];
      unpack8(h[x >> 1][x & 1], hf);
      unpack8(wv[x & 1], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float y = __fmul_rn(__fmul_rn(hf[e], rstd[x >> 1]), __fadd_rn(wf[e], 1.0f));
        o[e] = c == 1 ? __fadd_rn(o[e], y) : __fsub_rn(o[e], y);
      }
    }
    stg_stream(dst + rr * plane_stride, pack8(o));
  }
}

// --------------------------------------------------------- SwiGLU + planes
__device__ __forceinline__ float silu_f32(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// One thread per (row rho of a block row, 8-column vector of a plane).  Plane
// column l sits in chunk pair l / 64; its two S columns are 64 apart.
__global__ void __launch_bounds__(128)
k_swiglu_planes(const __nv_bfloat16* __restrict__ z, int64_t m2, int64_t inter, int64_t ldz,
                int rank, TermTable tt, __nv_bfloat16* __restrict__ out, int64_t ld_out) {
  const int64_t rho = blockIdx.x;
  const int64_t v = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
  const int64_t l = v * 8;
  if (l >= inter / 2) return;
  const int64_t c0 = (l / 64) * 128 + (l % 64);
  float s[4][8];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const __nv_bfloat16* row = z + (i * m2 + rho) * ldz;
      float g[8], u[8];
      unpack8(*reinterpret_cast<const Vec8*>(row + c0 + hh * 64), g);
      unpack8(*reinterpret_cast<const Vec8*>(row + inter + c0 + hh * 64), u);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[i * 2 + hh][e] = silu_f32(g[e]) * u[e];
    }
  for (int r = 0; r < rank; ++r) {
    float o[8];
    signed_sum(tt, r, s, o);
    *reinterpret_cast<Vec8*>(out + (r * m2 + rho) * ld_out + l) = pack8(o);
  }
}

// --------------------------------------------------------- dense-arm seams
__global__ void __launch_bounds__(1024)
k_add_rmsnorm(const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ residual,
              const __nv_bfloat16* __restrict__ norm_w, int64_t k, float eps,
              __nv_bfloat16* residual_out, __nv_bfloat16* __restrict__ x) {
  __shared__ float s_part[32];
  extern __shared__ __align__(16) unsigned char s_row_raw[];
  Vec8* s_row = reinterpret_cast<Vec8*>(s_row_raw);
  const int64_t row = blockIdx.x;
  const int64_t nvec = k / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  float ss = 0.f;
  for (int64_t v = tid; v < nvec; v += blockDim.x) {
    const int64_t off = row * k + v * 8;
    Vec8 hv = *reinterpret_cast<const Vec8*>(residual + off);      // no delta: h is the residual
    if (delta != nullptr) {
      float d[8], r[8], s[8];
      unpack8(*reinterpret_cast<const Vec8*>(delta + off), d);
      unpack8(hv, r);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] = d[e] + r[e];
      hv = pack8(s);
    }
    if (residual_out != nullptr) *reinterpret_cast<Vec8*>(residual_out + off) = hv;
    s_row[v] = hv;
    float hf[8];
    unpack8(hv, hf);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(hf[e], hf[e], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) s_part[warp] = ss;
  __syncthreads();
  float part = lane < nwarps ? s_part[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  const float rstd = rsqrtf(part / static_cast<float>(k) + eps);
  for (int64_t v = tid; v < nvec; v += blockDim.x) {
    float hf[8], w[8], y[8];
    unpack8(s_row[v], hf);
    unpack8(*reinterpret_cast<const Vec8*>(norm_w + v * 8), w);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = hf[e] * rstd * (w[e] + 1.0f);
    *reinterpret_cast<Vec8*>(x + row * k + v * 8) = pack8(y);
  }
}

// The same seam for rows of at most 1024 vectors (K <= 8192) and an even row count, in the style
// of the rank-7 arm's register kernel so that the two arms' norm kernels run at the same fraction
// of HBM: one CTA per pair of adjacent rows, one thread per vector of both rows, every load issued
// before anything is consumed, h kept packed in registers, streaming loads and stores.
__global__ void __launch_bounds__(1024)
k_add_rmsnorm_reg(const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ residual,
                  const __nv_bfloat16* __restrict__ norm_w, int k, float eps,
                  __nv_bfloat16* residual_out, __nv_bfloat16* __restrict__ x) {
  __shared__ float s_part[2][32];
  const int nvec = k / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const bool live = tid < nvec;
  const int v = live ? tid : 0;
  const size_t base = static_cast<size_t>(blockIdx.x) * 2 * k + v * 8;
  Vec8 h[2];
  if (delta != nullptr) {
    Vec8 d[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      d[i] = ldg_stream(delta + base + static_cast<size_t>(i) * k);
      h[i] = ldg_stream(residual + base + static_cast<size_t>(i) * k);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float df[8], rf[8], sf[8];
      unpack8(d[i], df);
      unpack8(h[i], rf);
#pragma unroll
      for (int e = 0; e < 8; ++e) sf[e] = df[e] + rf[e];
      h[i] = pack8(sf);
      if (live && residual_out != nullptr) stg_stream(residual_out + base + static_cast<size_t>(i) * k, h[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i) h[i] = ldg_stream(residual + base + static_cast<size_t>(i) * k);
  }
  float ss[2] = {0.f, 0.f};
  if (live) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float hf[8];
      unpack8(h[i], hf);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss[i] = fmaf(hf[e], hf[e], ss[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    if (lane == 0) s_part[i][warp] = ss[i];
  }
  __syncthreads();
  if (!live) return;
  float w[8];
  unpack8(*reinterpret_cast<const Vec8*>(norm_w + v * 8), w);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float part = lane < nwarps ? s_part[i][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const float rstd = rsqrtf(part / static_cast<float>(k) + eps);
    float hf[8], y[8];
    unpack8(h[i], hf);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = hf[e] * rstd * (w[e] + 1.0f);
    stg_stream(x + base + static_cast<size_t>(i) * k, pack8(y));
  }
}

__global__ void __launch_bounds__(256)
k_swiglu(const __nv_bfloat16* __restrict__ z, int64_t inter, int64_t ldz,
         __nv_bfloat16* __restrict__ s, int64_t lds) {
  const int64_t row = blockIdx.x;
  const int64_t v = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
  if (v * 8 >= inter) return;
  float g[8], u[8], o[8];
  unpack8(*reinterpret_cast<const Vec8*>(z + row * ldz + v * 8), g);
  unpack8(*reinterpret_cast<const Vec8*>(z + row * ldz + inter + v * 8), u);
#pragma unroll
  for (int e = 0; e < 8; ++e)
    o[e] = __bfloat162float(__float2bfloat16_rn(silu_f32(g[e]))) * u[e];
  *reinterpret_cast<Vec8*>(s + row * lds + v * 8) = pack8(o);
}

__global__ void __launch_bounds__(256)
k_add(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
      __nv_bfloat16* __restrict__ out, int64_t nvec) {
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float x[8], y[8], o[8];
    unpack8(reinterpret_cast<const Vec8*>(a)[v], x);
    unpack8(reinterpret_cast<const Vec8*>(b)[v], y);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = x[e] + y[e];
    reinterpret_cast<Vec8*>(out)[v] = pack8(o);
  }
}

TermTable a_table(const lcg_scheme* s) {
  TermTable t{};
  for (int r = 0; r < s->rank; ++r)
    for (int x = 0; x < 4; ++x) t.coef[r][x] = static_cast<float>(s->a[r][x]);
  return t;
}
TermTable b_table(const lcg_scheme* s) {
  TermTable t{};
  for (int r = 0; r < s->rank; ++r)
    for (int x = 0; x < 4; ++x) t.coef[r][x] = static_cast<float>(s->b[r][x]);
  return t;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_planes(const lcg_scheme* scheme, const void* src, int64_t rows, int64_t cols,
                  int64_t ld, bool b_side, void* out, int64_t ld_out, void* stream) {
  if (scheme == nullptr || src == nullptr || out == nullptr)
    return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (rows < 1 || cols < 1 || ld < cols) return fail(LCG_ERR_BAD_ARG, "bad extents");
  int64_t rows2, k2, k2p;
  lcg_plane_geometry(rows, cols, b_side ? 8 : 1, &rows2, &k2, &k2p);
  if (ld_out < k2p || ld_out % 8 != 0)
    return fail(LCG_ERR_BAD_ARG, "plane leading dimension %lld must be >= %lld and a multiple of 8",
                (long long)ld_out, (long long)k2p);
  if (!aligned16(out)) return fail(LCG_ERR_MISALIGNED, "plane buffer must be 16-byte aligned");
  if (rows2 > 0x7fffffffLL) return fail(LCG_ERR_UNSUPPORTED_SHAPE, "too many rows");
  const bool vec_ok = aligned16(src) && ld % 8 == 0 && k2 % 8 == 0;
  const int64_t nvec = k2p / 8;
  dim3 grid(static_cast<unsigned>(rows2), static_cast<unsigned>((nvec + 127) / 128));
  const TermTable table = b_side ? b_table(scheme) : a_table(scheme);
  // The A side runs per forward pass of the bare GEMM: compiled for the shipped tables.  (The B
  // side is the offline weight transform.)
  const unsigned long long code = b_side ? 0 : table_code(table, scheme->rank);
  auto kern = code == kCodePostsumA ? k_planes<kCodePostsumA>
              : code == kCodeLocalityA ? k_planes<kCodeLocalityA> : k_planes<0>;
  kern<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), rows, cols, ld, rows2, k2, k2p, scheme->rank, table,
      b_side, vec_ok, static_cast<__nv_bfloat16*>(out), ld_out);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

}  // namespace
}  // namespace lcg

using namespace lcg;

extern "C" int lcg_prepare_b(const lcg_scheme_t* scheme, const void* w, int64_t N, int64_t K,
                             int64_t ldw, void* out, int64_t ld_out, void* stream) {
  return launch_planes(scheme, w, N, K, ldw, true, out, ld_out, stream);
}

extern "C" int lcg_a_planes(const lcg_scheme_t* scheme, const void* a, int64_t M, int64_t K,
                            int64_t lda, void* out, int64_t ld_out, void* stream) {
  return launch_planes(scheme, a, M, K, lda, false, out, ld_out, stream);
}

extern "C" int lcg_norm_planes(const lcg_scheme_t* scheme, const void* delta, const void* residual,
                               const void* norm_weight, int64_t M, int64_t K, float eps,
                               void* residual_out, void* out, int64_t ld_out, void* stream) {
  if (!scheme || !residual || !norm_weight || !out || (delta && !residual_out))
    return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (!delta) residual_out = nullptr;       // no delta: the residual stream is the input, nothing is stored
  if (M < 2 || M % 2 != 0 || K < 16 || K % 16 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE,
                "fused norm needs an even M and K %% 16 == 0, got M=%lld K=%lld", (long long)M,
                (long long)K);
  if ((delta && !aligned16(delta)) || !aligned16(residual) || !aligned16(norm_weight) ||
      (residual_out && !aligned16(residual_out)) || !aligned16(out))
    return fail(LCG_ERR_MISALIGNED, "all operands must be 16-byte aligned");
  const int64_t k2p = (K / 2 + 63) / 64 * 64;
  if (ld_out < k2p || ld_out % 8 != 0)
    return fail(LCG_ERR_BAD_ARG, "plane leading dimension %lld must be >= %lld and a multiple of 8",
                (long long)ld_out, (long long)k2p);
  const int64_t nvec_p = k2p / 8;
  // Register forms: a shipped table and rows of at most 512 vectors per block column.  The lean
  // one takes the rows too wide for the other and every call without a delta.
  if (k2p == K / 2 && K / 16 <= 512 && M / 2 <= 0x7fffffff && ld_out <= 0x7fffffff) {
    const TermTable table = a_table(scheme);
    const unsigned long long code = table_code(table, scheme->rank);
    if (code == kCodePostsumA || code == kCodeLocalityA) {
      const int nvec = static_cast<int>(K / 16);
      const int threads = (nvec + 31) / 32 * 32;
      const bool postsum = code == kCodePostsumA;
      auto kern = postsum ? k_norm_planes_reg<kCodePostsumA> : k_norm_planes_reg<kCodeLocalityA>;
      if (!delta)
        kern = postsum ? k_norm_planes_lean<kCodePostsumA, false> : k_norm_planes_lean<kCodeLocalityA, false>;
      else if (nvec > 416)
        kern = postsum ? k_norm_planes_lean<kCodePostsumA, true> : k_norm_planes_lean<kCodeLocalityA, true>;
      kern<<<static_cast<unsigned>(M / 2), threads, 0, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(residual),
          static_cast<const __nv_bfloat16*>(norm_weight), static_cast<int>(M / 2), static_cast<int>(K), eps,
          static_cast<__nv_bfloat16*>(residual_out), static_cast<__nv_bfloat16*>(out), static_cast<int>(ld_out));
      LCG_CUDA_OK(cudaGetLastError());
      count_launch();
      return LCG_OK;
    }
  }
  // Staged form: whole row pair in shared memory, when it fits three CTAs to an SM.
  if (k2p == K / 2 && 8 * K <= 72 * 1024 && M / 2 <= 0x7fffffff && ld_out <= 0x7fffffff) {
    const int nvec = static_cast<int>(K / 16);
    const int threads = nvec >= 512 ? 512 : (nvec + 31) / 32 * 32;
    const size_t smem = static_cast<size_t>(8) * K;
    static bool configured[64] = {};
    int dev = 0;
    LCG_CUDA_OK(cudaGetDevice(&dev));
    const TermTable table = a_table(scheme);
    const unsigned long long code = table_code(table, scheme->rank);
    auto kern = code == kCodePostsumA    ? k_norm_planes_staged<kCodePostsumA>
                : code == kCodeLocalityA ? k_norm_planes_staged<kCodeLocalityA>
                                         : k_norm_planes_staged<0>;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      LCG_CUDA_OK(cudaFuncSetAttribute(k_norm_planes_staged<kCodePostsumA>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
      LCG_CUDA_OK(cudaFuncSetAttribute(k_norm_planes_staged<kCodeLocalityA>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
      LCG_CUDA_OK(cudaFuncSetAttribute(k_norm_planes_staged<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       72 * 1024));
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kern<<<static_cast<unsigned>(M / 2), threads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(residual),
        static_cast<const __nv_bfloat16*>(norm_weight), static_cast<int>(M / 2), static_cast<int>(K), eps,
        scheme->rank, table, static_cast<__nv_bfloat16*>(residual_out),
        static_cast<__nv_bfloat16*>(out), static_cast<int>(ld_out));
    LCG_CUDA_OK(cudaGetLastError());
    count_launch();
    return LCG_OK;
  }
  int vpt = 1;
  while ((nvec_p + vpt - 1) / vpt > 1024) vpt *= 2;
  if (vpt > 4) return fail(LCG_ERR_UNSUPPORTED_SHAPE, "K=%lld too wide for the fused norm", (long long)K);
  const int threads = static_cast<int>(((nvec_p + vpt - 1) / vpt + 31) / 32 * 32);
  const TermTable tt = a_table(scheme);
  auto st = static_cast<cudaStream_t>(stream);
  auto d = static_cast<const __nv_bfloat16*>(delta);
  auto r = static_cast<const __nv_bfloat16*>(residual);
  auto w = static_cast<const __nv_bfloat16*>(norm_weight);
  auto ro = static_cast<__nv_bfloat16*>(residual_out);
  auto o = static_cast<__nv_bfloat16*>(out);
  const unsigned grid = static_cast<unsigned>(M / 2);
  if (vpt == 1)
    k_norm_planes<1><<<grid, threads, 0, st>>>(d, r, w, M / 2, K, k2p, eps, scheme->rank, tt, ro, o, ld_out);
  else if (vpt == 2)
    k_norm_planes<2><<<grid, threads, 0, st>>>(d, r, w, M / 2, K, k2p, eps, scheme->rank, tt, ro, o, ld_out);
  else
    k_norm_planes<4><<<grid, threads, 0, st>>>(d, r, w, M / 2, K, k2p, eps, scheme->rank, tt, ro, o, ld_out);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

extern "C" int lcg_swiglu_planes(const lcg_scheme_t* plane_scheme, const void* z, int64_t M,
                                 int64_t I, int64_t ldz, void* out, int64_t ld_out, void* stream) {
  if (!plane_scheme || !z || !out) return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (M < 2 || M % 2 != 0 || I < 128 || I % 128 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE,
                "the interleaved gauge needs an even M and I %% 128 == 0, got M=%lld I=%lld",
                (long long)M, (long long)I);
  if (ldz < 2 * I || ldz % 8 != 0 || ld_out < I / 2 || ld_out % 8 != 0)
    return fail(LCG_ERR_BAD_ARG, "bad leading dimensions");
  if (!aligned16(z) || !aligned16(out)) return fail(LCG_ERR_MISALIGNED, "operands must be 16-byte aligned");
  const int64_t nvec = I / 2 / 8;
  dim3 grid(static_cast<unsigned>(M / 2), static_cast<unsigned>((nvec + 127) / 128));
  k_swiglu_planes<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(z), M / 2, I, ldz, plane_scheme->rank, a_table(plane_scheme),
      static_cast<__nv_bfloat16*>(out), ld_out);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

extern "C" int lcg_add_rmsnorm(const void* delta, const void* residual, const void* norm_weight,
                               int64_t M, int64_t K, float eps, void* residual_out, void* x,
                               void* stream) {
  if (!residual || !norm_weight || !x || (delta && !residual_out))
    return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (!delta) residual_out = nullptr;       // no delta: the residual stream is the input, nothing is stored
  if (M < 1 || K < 8 || K % 8 != 0 || K > 24576)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "needs K %% 8 == 0 and K <= 24576, got K=%lld", (long long)K);
  if ((delta && !aligned16(delta)) || !aligned16(residual) || !aligned16(norm_weight) ||
      (residual_out && !aligned16(residual_out)) || !aligned16(x))
    return fail(LCG_ERR_MISALIGNED, "all operands must be 16-byte aligned");
  const int64_t nvec = K / 8;
  const int threads = static_cast<int>(nvec >= 1024 ? 1024 : (nvec + 31) / 32 * 32);
  if (nvec <= 1024 && M % 2 == 0 && M / 2 <= 0x7fffffff) {
    k_add_rmsnorm_reg<<<static_cast<unsigned>(M / 2), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(residual),
        static_cast<const __nv_bfloat16*>(norm_weight), static_cast<int>(K), eps,
        static_cast<__nv_bfloat16*>(residual_out), static_cast<__nv_bfloat16*>(x));
    LCG_CUDA_OK(cudaGetLastError());
    count_launch();
    return LCG_OK;
  }
  k_add_rmsnorm<<<static_cast<unsigned>(M), threads, static_cast<size_t>(K) * 2,
                  static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(norm_weight), K, eps,
      static_cast<__nv_bfloat16*>(residual_out), static_cast<__nv_bfloat16*>(x));
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

extern "C" int lcg_swiglu(const void* z, int64_t M, int64_t I, int64_t ldz, void* s, int64_t lds,
                          void* stream) {
  if (!z || !s) return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (M < 1 || I < 8 || I % 8 != 0 || ldz < 2 * I || ldz % 8 != 0 || lds < I || lds % 8 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "needs I %% 8 == 0 and 16-byte aligned rows");
  if (!aligned16(z) || !aligned16(s)) return fail(LCG_ERR_MISALIGNED, "operands must be 16-byte aligned");
  const int64_t nvec = I / 8;
  dim3 grid(static_cast<unsigned>(M), static_cast<unsigned>((nvec + 255) / 256));
  k_swiglu<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(z), I, ldz, static_cast<__nv_bfloat16*>(s), lds);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

extern "C" int lcg_add(const void* a, const void* b, void* out, int64_t n, void* stream) {
  if (!a || !b || !out) return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (n < 8 || n % 8 != 0) return fail(LCG_ERR_UNSUPPORTED_SHAPE, "n must be a positive multiple of 8");
  if (!aligned16(a) || !aligned16(b) || !aligned16(out))
    return fail(LCG_ERR_MISALIGNED, "operands must be 16-byte aligned");
  const int64_t nvec = n / 8;
  const unsigned grid = static_cast<unsigned>(nvec / 256 + 1 < 148 * 8 ? nvec / 256 + 1 : 148 * 8);
  k_add<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
      static_cast<__nv_bfloat16*>(out), nvec);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}
