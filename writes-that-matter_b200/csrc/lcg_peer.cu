// Tensor-parallel exchange over peer memory (NVLink / NVSwitch): the barrier between ranks and
// the kernel that finishes the row-parallel `down` projection -- reduce the partials the ranks'
// GEMM kernels pushed into this rank's slots, add the residual, and store the finished rows into
// every rank's output.  Plain peer loads and stores only (no multimem, no TMA).
//
// The reference is single-GPU (lcgemm/integrate/qwen_patch.py:216-217 refuses TP > 1); these
// entry points have no counterpart there.
#include <cuda_bf16.h>

#include "lcg_common.h"

namespace lcg {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kCodeBarrier = 106;

struct BarrierArgs {
  uint32_t* flags[kMaxWorld];   // flags[r]: rank r's flag array (2 * kMaxWorld words), peer-mapped
  int32_t world, rank;
  uint32_t epoch;
  int32_t* status;
  uint64_t limit_ns;
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One CTA; thread t tells rank t "rank `rank` has reached barrier `epoch`" and then waits until
// rank t has said the same here.  Epochs only grow, so a flag that is already ahead passes.
// The wait is bounded: when it runs out the kernel records kCodeBarrier and returns.
__global__ void k_peer_barrier(const BarrierArgs a) {
  __shared__ uint32_t s_epoch;
  const int t = static_cast<int>(threadIdx.x);
  // Epoch 0 in the arguments: count the calls on the device (word kMaxWorld of this rank's own
  // array), so that the same launch can be replayed from a CUDA graph.
  if (t == 0) s_epoch = a.epoch != 0u ? a.epoch : atomicAdd(a.flags[a.rank] + kMaxWorld, 1u) + 1u;
  __syncthreads();
  if (t >= a.world) return;
  const uint32_t epoch = s_epoch;
  __threadfence_system();
  st_release_sys(a.flags[t] + a.rank, epoch);
  const uint32_t* mine = a.flags[a.rank] + t;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
    __nanosleep(100);
    if ((++spins & 0x3fu) == 0 && globaltimer_ns() - t0 > a.limit_ns) {
      if (a.status != nullptr) atomicCAS(a.status, 0, kCodeBarrier);
      return;
    }
  }
}

struct GatherArgs {
  const __nv_bfloat16* slots;   // (world, rows_per_owner, cols): what each rank pushed for my rows
  const __nv_bfloat16* h;       // (m, cols) residual, leading dimension ld_h
  int64_t ld_h;
  __nv_bfloat16* out[kMaxWorld];   // every rank's (m, cols) output, contiguous
  int32_t world, rank;
  int64_t m, cols, rows_per_owner;
};

__device__ __forceinline__ void add8(const uint4& q, float (&acc)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(w[i] << 16);
    acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
  }
}

// out[rank's rows] = bf16(h + sum_w slots[w]) in fp32, ranks summed in index order, stored into
// all ranks' outputs (the all-gather half).  One 16-byte vector per thread and iteration.
__global__ void __launch_bounds__(256) k_reduce_gather(const __grid_constant__ GatherArgs a) {
  const int64_t vec_per_row = a.cols / 8;
  const int64_t row0 = static_cast<int64_t>(a.rank) * a.rows_per_owner;
  const int64_t rows = min(a.rows_per_owner, a.m - row0);
  const int64_t nvec = rows * vec_per_row;
  const int64_t slot_stride = a.rows_per_owner * a.cols;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t lr = v / vec_per_row;
    const int64_t c = (v - lr * vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    uint4 q[kMaxWorld];
#pragma unroll
    for (int w = 0; w < kMaxWorld; ++w)
      if (w < a.world)
        q[w] = __ldcs(reinterpret_cast<const uint4*>(a.slots + w * slot_stride + lr * a.cols + c));
    add8(__ldg(reinterpret_cast<const uint4*>(a.h + (row0 + lr) * a.ld_h + c)), acc);
#pragma unroll
    for (int w = 0; w < kMaxWorld; ++w)
      if (w < a.world) add8(q[w], acc);
    uint4 o;
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0], acc[1]);
    const __nv_bfloat162 p1 = __floats2bfloat162_rn(acc[2], acc[3]);
    const __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4], acc[5]);
    const __nv_bfloat162 p3 = __floats2bfloat162_rn(acc[6], acc[7]);
    o.x = *reinterpret_cast<const uint32_t*>(&p0);
    o.y = *reinterpret_cast<const uint32_t*>(&p1);
    o.z = *reinterpret_cast<const uint32_t*>(&p2);
    o.w = *reinterpret_cast<const uint32_t*>(&p3);
    // Peers in the order rank + 1, rank + 2, ..., own copy last: the ranks run this kernel at the
    // same time, and all of them storing to peer 0 first, then peer 1, would crowd one link at a time.
    const int64_t off = (row0 + lr) * a.cols + c;
#pragma unroll
    for (int j = 1; j <= kMaxWorld; ++j)
      if (j <= a.world) {
        int w = a.rank + j;
        if (w >= a.world) w -= a.world;
        __stcg(reinterpret_cast<uint4*>(a.out[w] + off), o);
      }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace lcg

using namespace lcg;

extern "C" int lcg_peer_barrier(void* const* flags, int world, int rank, uint32_t epoch,
                                int64_t limit_us, int32_t* status, void* stream) {
  if (!flags) return fail(LCG_ERR_BAD_ARG, "NULL flag table");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return fail(LCG_ERR_BAD_ARG, "world must be 1..%d and rank inside it; got world=%d rank=%d",
                kMaxWorld, world, rank);
  if (limit_us < 1 || limit_us > 60 * 1000 * 1000)
    return fail(LCG_ERR_BAD_ARG, "limit_us must be in [1, 60e6]");
  BarrierArgs a{};
  for (int w = 0; w < world; ++w) {
    if (!flags[w] || (reinterpret_cast<uintptr_t>(flags[w]) & 3u) != 0)
      return fail(LCG_ERR_BAD_ARG, "flag pointer %d is NULL or unaligned", w);
    a.flags[w] = static_cast<uint32_t*>(flags[w]);
  }
  a.world = world;
  a.rank = rank;
  a.epoch = epoch;
  a.status = status;
  a.limit_ns = static_cast<uint64_t>(limit_us) * 1000ull;
  k_peer_barrier<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}

extern "C" int lcg_reduce_gather(const void* slots, const void* h, int64_t ld_h, void* const* outs,
                                 int64_t M, int64_t cols, int64_t rows_per_owner, int world,
                                 int rank, void* stream) {
  if (!slots || !h || !outs) return fail(LCG_ERR_BAD_ARG, "NULL argument");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return fail(LCG_ERR_BAD_ARG, "world must be 1..%d and rank inside it; got world=%d rank=%d",
                kMaxWorld, world, rank);
  if (M < 1 || cols < 8 || cols % 8 != 0 || ld_h < cols || ld_h % 8 != 0)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE, "needs cols %% 8 == 0 and ld_h %% 8 == 0, ld_h >= cols");
  if (rows_per_owner < 1 || rows_per_owner * world < M)
    return fail(LCG_ERR_BAD_ARG, "rows_per_owner * world must cover M");
  if (!aligned16(slots) || !aligned16(h)) return fail(LCG_ERR_MISALIGNED, "operands must be 16-byte aligned");
  GatherArgs a{};
  for (int w = 0; w < world; ++w) {
    if (!outs[w] || !aligned16(outs[w])) return fail(LCG_ERR_MISALIGNED, "output %d is NULL or unaligned", w);
    a.out[w] = static_cast<__nv_bfloat16*>(outs[w]);
  }
  a.slots = static_cast<const __nv_bfloat16*>(slots);
  a.h = static_cast<const __nv_bfloat16*>(h);
  a.ld_h = ld_h;
  a.world = world;
  a.rank = rank;
  a.m = M;
  a.cols = cols;
  a.rows_per_owner = rows_per_owner;
  const int64_t row0 = static_cast<int64_t>(rank) * rows_per_owner;
  if (row0 >= M) return LCG_OK;   // this rank owns no rows
  const int64_t rows = rows_per_owner < M - row0 ? rows_per_owner : M - row0;
  const int64_t nvec = rows * (cols / 8);
  const int64_t want = (nvec + 255) / 256;
  const unsigned grid = static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8);
  k_reduce_gather<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LCG_CUDA_OK(cudaGetLastError());
  count_launch();
  return LCG_OK;
}
