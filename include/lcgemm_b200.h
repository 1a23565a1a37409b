/*
 * lcgemm_b200 -- C ABI of the B200 (sm_100a) rank-7 bilinear GEMM path.
 *
 * The reference project (lcgemm) has no native layer: its device code is
 * generated from Python at run time and its seams call compiled callables with
 * wrapped tensors (lcgemm/seams/gate_up.py:107-127, lcgemm/seams/down.py:88-102).
 * The functions below are what a binding for that path would call instead.
 * Every entry point
 *   - takes plain device pointers, extents, leading dimensions (in elements)
 *     and the CUDA stream as `void*` (a cudaStream_t / CUstream);
 *   - never allocates, frees or synchronises; all launches are asynchronous
 *     on the given stream;
 *   - returns LCG_OK (0) or a negative LCG_ERR_* code, with the text of the
 *     last failure of the calling thread available from lcg_last_error().
 *
 * Conventions (the reference's, lcgemm/kernels/sm100.py:3-5): all matrices
 * are bf16, row-major; activations are (M, K); weights are (N, K) "K-major",
 * the layout torch.nn.functional.linear stores; accumulation is fp32.
 *
 * Plane geometry.  A one-level 2x2x2 scheme splits M, K, N in two blocks.
 *   M2  = ceil(M / 2)                       rows of one A block
 *   N2  = round_up(ceil(N / 2), 8)          rows of one B block (and the column
 *                                           offset of C block j is j * N2)
 *   K2  = ceil(K / 2),  K2p = round_up(K2, 64)
 * A planes are a (rank * M2, K2p) matrix, plane r at row r * M2;
 * B planes are a (rank * N2, K2p) matrix, plane r at row r * N2.  Elements that
 * fall outside the source matrix, and columns K2..K2p, are zero.  For the
 * shapes the reference supports (everything divisible) these are exactly the
 * reference's (R * M/p, K/q) and (R * N/s, K/q) planes (lcgemm/planes.py:54-71,
 * lcgemm/seams/gate_up.py:82-93).  lcg_plane_geometry() returns the numbers.
 *
 * Device status word.  The tcgen05 kernels bound every wait on an mbarrier;
 * a wait that runs out writes a nonzero code into `status` (one int32 in
 * device memory, zeroed by the caller before the first launch) and lets the
 * kernel run to its end without blocking again.  `status` may be NULL.
 */
#ifndef LCGEMM_B200_H
#define LCGEMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LCG_OK                      0
#define LCG_ERR_BAD_ARG           (-1)
#define LCG_ERR_UNSUPPORTED_SHAPE (-2)
#define LCG_ERR_MISALIGNED        (-3)
#define LCG_ERR_SCHEME            (-4)
#define LCG_ERR_CUDA              (-5)
#define LCG_ERR_DEVICE_TIMEOUT    (-6)

/* Work decomposition of the rank-7 GEMM. */
#define LCG_SCHEDULE_ALL_RANKS   0  /* one CTA group walks all products of a tile;
                                       first write to a C block is a store, later
                                       ones reduce-adds (lcgemm/kernels/sm100.py:10-16,
                                       lcgemm/kernels/down.py:490-505) */
#define LCG_SCHEDULE_RANK_SPLIT  1  /* one (product, tile) unit per step, every
                                       contribution is a reduce-add into a C that
                                       arrives zeroed (lcgemm/kernels/down_rank_split.py:106-113,209-216) */

#define LCG_SCHEDULE_HYBRID      2  /* whole waves of tiles walk all products; the tiles of
                                       the last partial wave are split by product over all
                                       CTA groups (their C blocks are cleared by a small
                                       kernel first, then receive reduce-adds only).  Takes
                                       the place of the reference's two-region tail
                                       re-tiling (lcgemm/kernels/hetero.py:37-44) */

/* MMA pairing: 1 = one CTA per 128x256 tile, 2 = a 2-CTA pair per 256x256 tile
 * (the reference's tcgen05 CtaGroup.TWO, lcgemm/kernels/sm100.py:186-191). */
#define LCG_CTA_GROUP_DEFAULT 0

typedef struct lcg_scheme lcg_scheme_t;

/* ---- library ----------------------------------------------------------- */

int lcg_version(void);

/* Text of the calling thread's last failure ("" if none). Never NULL. */
const char* lcg_last_error(void);

/* ---- scheme (replaces lcgemm/scheme.py:121-486 on the native side) ------ */

/* Build a scheme handle from the coefficient tables of a 2x2x2 decomposition:
 * a, b, c are rank x 4 row-major over (i,k), (k,j), (i,j); `clear` is the
 * per-step accumulator-chain flag of a postsum plan or NULL for the plain
 * scatter epilogue (lcgemm/scheme.py:136-139,189-201).  The exact integer
 * tensor identity (lcgemm/scheme.py:324-361) and the chain plan
 * (lcgemm/scheme.py:363-408) are validated here as well; a scheme that fails
 * returns LCG_ERR_SCHEME. */
int lcg_scheme_create(const int8_t* a, const int8_t* b, const int8_t* c,
                      int rank, const int8_t* clear, lcg_scheme_t** out);
void lcg_scheme_destroy(lcg_scheme_t* scheme);

/* The derived epilogue plan, for cross-checking against the host-side Scheme
 * (lcgemm/scheme.py:250-264 `epi_groups`).  Writes, per step, up to 4 records
 * (bi, bj, coeff, is_first) into out[step*16 + 4*n ..]; counts[step] receives
 * the number of records. */
int lcg_scheme_plan(const lcg_scheme_t* scheme, int8_t* out, int32_t* counts);

/* ---- geometry ---------------------------------------------------------- */

/* rows2 = ceil(rows/2) rounded up to `row_align` (1 for A, 8 for B);
 * k2 = ceil(cols/2); k2p = round_up(k2, 64). */
int lcg_plane_geometry(int64_t rows, int64_t cols, int row_align,
                       int64_t* rows2, int64_t* k2, int64_t* k2p);

/* ---- operand planes ----------------------------------------------------- */

/* B planes of a static weight, fp32 sum and one rounding
 * (lcgemm/planes.py:54-71 `prepare_b`).  w is (N, K) with leading dimension
 * ldw; out is (rank * N2, ld_out) with ld_out >= K2p. */
int lcg_prepare_b(const lcg_scheme_t* scheme, const void* w, int64_t N, int64_t K,
                  int64_t ldw, void* out, int64_t ld_out, void* stream);

/* A planes of a plain activation matrix (no counterpart is shipped by the
 * reference, which removed its standalone A transform, lcgemm/planes.py:16-17;
 * semantics are those of lcgemm/chain_gauge.py:91-98 without SwiGLU or gauge).
 * a is (M, K) with leading dimension lda; out is (rank * M2, ld_out). */
int lcg_a_planes(const lcg_scheme_t* scheme, const void* a, int64_t M, int64_t K,
                 int64_t lda, void* out, int64_t ld_out, void* stream);

/* Fused residual add + RMSNorm + A planes
 * (lcgemm/kernels/fused_norm.py:140-198 `fused_norm_residual_kernel`):
 *   h = bf16(float(delta) + float(residual))      -> residual_out (may alias residual)
 *   y = float(h) * rsqrt(mean(h^2) + eps) * (float(norm_weight) + 1)
 *   out plane r = bf16(signed sum of the four blocks of y)
 * delta, residual, residual_out are contiguous (M, K); needs M even, K % 16 == 0.
 * delta may be NULL (the first layer of a stack, or a layer called on its own): then h is the
 * residual itself, one operand less is read and residual_out is neither needed nor written. */
int lcg_norm_planes(const lcg_scheme_t* scheme, const void* delta, const void* residual,
                    const void* norm_weight, int64_t M, int64_t K, float eps,
                    void* residual_out, void* out, int64_t ld_out, void* stream);

/* SwiGLU + the consumer's A planes in the interleaved-K gauge, as a kernel of
 * its own (lcgemm/chain_gauge.py:82-99 `chain_a_planes`; on the device the
 * reference fuses this into its GEMM, lcgemm/kernels/sm100.py:820-888).
 * z is (M, 2*I) = [gate | up] with leading dimension ldz; out is
 * (rank * M/2, I/2).  Needs M even and I % 128 == 0. */
int lcg_swiglu_planes(const lcg_scheme_t* plane_scheme, const void* z, int64_t M,
                      int64_t I, int64_t ldz, void* out, int64_t ld_out, void* stream);

/* ---- GEMMs --------------------------------------------------------------- */

/* Dense C = A @ B^T on tcgen05 (the baseline arm: what the stock model's
 * cuBLAS GEMM computes, lcgemm/integrate/qwen_patch.py:53-57).  A (M, K),
 * B (N, K), C (M, N); lda, ldb, ldc multiples of 8; K multiple of 8. */
int lcg_gemm_dense(const void* a, int64_t lda, const void* b, int64_t ldb,
                   void* c, int64_t ldc, int64_t M, int64_t N, int64_t K,
                   int cta_group, int32_t* status, void* stream);

/* Rank-7 C = A @ B^T from prepared planes
 * (lcgemm/kernels/sm100.py:447-752 mainloop + scatter, lcgemm/kernels/down.py,
 * lcgemm/kernels/down_rank_split.py).  With LCG_SCHEDULE_RANK_SPLIT the caller
 * passes C zeroed.  ldc multiple of 8. */
int lcg_gemm_r7(const lcg_scheme_t* scheme, const void* a_planes, int64_t ld_a,
                const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                int64_t M, int64_t N, int64_t K, int schedule, int cta_group,
                int32_t* status, void* stream);

/* Rank-7 C = A @ B^T straight from the activation matrix: the A operand of every product is
 * formed inside the GEMM kernel, on its way into shared memory, so no A planes exist in global
 * memory and the call needs no scratch.  Takes the place of the plane loads of the reference's
 * mainloop (lcgemm/kernels/sm100.py:578-592) and of the plane-forming pass in front of it
 * (lcgemm/planes.py:27-50 `apply_terms`): a product whose A row is a single block with
 * coefficient +1 is loaded by TMA from that block; a product with two terms goes through eight
 * producer warps (16-byte loads of both blocks, one packed bf16 add or subtract -- the fp32 sum
 * rounded once -- swizzled stores into the operand stage).  The result equals lcg_a_planes +
 * lcg_gemm_r7 with the same schedule bit for bit when the schedule is LCG_SCHEDULE_ALL_RANKS.
 * Needs K % 128 == 0 and a scheme whose A rows have one or two +-1 terms
 * (2x2_locality_ordered); anything else returns LCG_ERR_UNSUPPORTED_SHAPE / LCG_ERR_SCHEME and
 * the caller uses the plane path.  a is (M, K) with lda % 8 == 0, 16-byte aligned. */
int lcg_gemm_r7_fused(const lcg_scheme_t* scheme, const void* a, int64_t lda,
                      const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                      int64_t M, int64_t N, int64_t K, int schedule, int cta_group,
                      int32_t* status, void* stream);
/* 1 when lcg_gemm_r7_fused accepts this scheme and shape, else 0. */
int lcg_gemm_r7_fused_supported(const lcg_scheme_t* scheme, int64_t M, int64_t N, int64_t K);

/* Rank-7 C = A @ B^T from the activation matrix with the plane-forming pass folded into the
 * GEMM kernel: while the MMAs work on one product, eight otherwise idle warps of every CTA form
 * the A plane of the next two-term product (16-byte loads of its two blocks, one packed bf16 add
 * or subtract, 16-byte stores) into `scratch`, from where the TMA producer loads it, L2-hot, once
 * a chunk counter says the plane is whole; products whose A row is a single block with
 * coefficient +1 are loaded from `a` itself.  Same arithmetic and rounding as lcg_a_planes +
 * lcg_gemm_r7 (bit-equal with LCG_SCHEDULE_ALL_RANKS), without the separate pass in front of the
 * GEMM that those two pay for (lcgemm/planes.py:27-50, lcgemm/kernels/sm100.py:578-592).
 * A scheme whose first products are single-block ones (2x2_locality_lead_single) starts without
 * waiting.  scratch: lcg_gemm_r7_ahead_scratch_bytes() bytes, 256-byte aligned, owned by the
 * caller; the first 256 bytes are cleared on the stream by this call.  Needs K % 128 == 0, A-side
 * rows of one or two +-1 terms, a 16-byte aligned with lda % 8 == 0.  All waits are bounded
 * (status code 107: a plane never became whole). */
int lcg_gemm_r7_ahead(const lcg_scheme_t* scheme, const void* a, int64_t lda,
                      const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                      int64_t M, int64_t N, int64_t K, void* scratch, int64_t scratch_bytes,
                      int schedule, int cta_group, int32_t* status, void* stream);
/* Bytes of scratch lcg_gemm_r7_ahead needs, or -1 when it does not take this scheme / shape. */
int64_t lcg_gemm_r7_ahead_scratch_bytes(const lcg_scheme_t* scheme, int64_t M, int64_t K);

/* lcg_gemm_r7 restricted to the tile rows [tile_row_begin, tile_row_end) of both block rows
 * (a tile row is 128 * cta_group rows of a block row: output rows i * M2 + [begin, end) * 256
 * for i = 0, 1 with the default pairing; tile_row_end < 0 means "to the last"), on at most
 * `max_groups` CTA groups (0 = all SMs).  This is how the tensor-parallel layer pipelines the
 * row-parallel `down` GEMM with the all-reduce of the slab before it: the slabs run back to
 * back on the compute stream while NCCL reduces finished slabs on the SMs left free.  No
 * counterpart in the reference, which is single-GPU (lcgemm/integrate/qwen_patch.py:216-217). */
int lcg_gemm_r7_slab(const lcg_scheme_t* scheme, const void* a_planes, int64_t ld_a,
                     const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                     int64_t M, int64_t N, int64_t K, int schedule, int cta_group,
                     int tile_row_begin, int tile_row_end, int max_groups,
                     int32_t* status, void* stream);

/* The chained gate_up GEMM (lcgemm/kernels/sm100.py `LcGemmSm100.call_planes`):
 * Z = rank-7 product into z (M, N = 2*I), then, in the same kernel, one tile
 * behind the mainloop, S = silu(Z[:, :I]) * Z[:, I:] and the consumer's A planes
 * L_r(S) in the interleaved gauge into down_planes (plane_rank * M/2, I/2);
 * optionally zeroes `preclear` (preclear_bytes, multiple of 16) for a
 * rank-split consumer (lcgemm/kernels/sm100.py:779-815).
 * `schedule` is LCG_SCHEDULE_ALL_RANKS or LCG_SCHEDULE_HYBRID; with the hybrid schedule the
 * tail tiles' seven products come from different CTAs, so their SwiGLU/plane phase runs in a
 * small second kernel queued behind the GEMM on the same stream (the library keeps no state
 * between launches).
 * Needs M % 2 == 0, N % 256 == 0, K % 128 == 0. */
int lcg_gate_up_chain(const lcg_scheme_t* scheme, const lcg_scheme_t* plane_scheme,
                      const void* a_planes, int64_t ld_a, const void* b_planes, int64_t ld_b,
                      void* z, int64_t ldz, int64_t M, int64_t N, int64_t K,
                      void* down_planes, int64_t ld_planes,
                      void* preclear, int64_t preclear_bytes, int schedule, int cta_group,
                      int32_t* status, void* stream);

/* The same kernel with the residual add of `down` folded into the chain.  No counterpart in the
 * reference, whose `down` kernels have no residual operand: it leaves the add to the next layer's
 * fused norm kernel (lcgemm/integrate/qwen_patch.py:160-167).  Instead of zeroing the rank-split consumer's output,
 * the plane warps copy `init_from` (consumer_bytes, same layout as consumer_out, not overlapping
 * it) into it, so every contribution the consumer reduce-adds lands on the residual stream and
 * `consumer_out` ends as residual + down(...) without a separate add kernel.  Each contribution is
 * then rounded to bf16 at the residual's magnitude instead of the branch's: see the numerics notes
 * of the package before switching it on. */
int lcg_gate_up_chain_init(const lcg_scheme_t* scheme, const lcg_scheme_t* plane_scheme,
                           const void* a_planes, int64_t ld_a, const void* b_planes, int64_t ld_b,
                           void* z, int64_t ldz, int64_t M, int64_t N, int64_t K,
                           void* down_planes, int64_t ld_planes,
                           void* consumer_out, int64_t consumer_bytes, const void* init_from,
                           int schedule, int cta_group, int32_t* status, void* stream);

/* ---- tensor parallel over peer memory (NVLink / NVSwitch) ------------------
 * The reference runs on one GPU (lcgemm/integrate/qwen_patch.py:216-217 refuses TP > 1);
 * the three entry points below have no counterpart there.  One process per GPU; the caller
 * exchanges device pointers of peer-mapped buffers (CUDA IPC or symmetric memory) once.
 *
 * lcg_gemm_r7_push: the row-parallel `down` projection of one rank.  Rank-7 C = A @ B^T from
 * prepared planes into this rank's partial `c` (M, N) with the hybrid schedule, and, in the
 * same kernel, one tile behind the mainloop, every finished tile is copied to the rank that
 * owns its rows: row g belongs to rank g / rows_per_owner and lands in slots[owner], an
 * (rows_per_owner, N) row-major region of the owner's memory reserved for this rank
 * (slots is a host array of `world` device pointers; slots[rank] is local).  The tail tiles
 * of the hybrid schedule are pushed by a small second kernel behind the GEMM.  Rank r starts its
 * walk over the tile rows r / world of the way down (and wraps), so that the ranks, which run this
 * kernel together, push to different owners at any moment instead of all to the same two.  N % 8 == 0,
 * c 16-byte aligned, ldc % 8 == 0, world <= 8. */
int lcg_gemm_r7_push(const lcg_scheme_t* scheme, const void* a_planes, int64_t ld_a,
                     const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                     int64_t M, int64_t N, int64_t K, void* const* slots, int world, int rank,
                     int64_t rows_per_owner, int cta_group, int32_t* status, void* stream);

/* Barrier between the ranks, on the stream: flags is a host array of `world` device pointers,
 * flags[r] = rank r's array of 16 uint32 words (zero before the first barrier), peer-mapped.
 * Rank `rank` writes `epoch` into word `rank` of every rank's array and waits until its own
 * array holds `epoch` or more in every word; epochs must grow from call to call.  With
 * epoch = 0 the kernel counts the calls itself (in word 8 of the rank's own array; every rank
 * must then use 0 for every barrier), which lets a CUDA graph replay the launch.  The wait
 * is bounded by limit_us: when it runs out the kernel writes 106 into `status` (may be NULL)
 * and returns, and the context stays usable. */
int lcg_peer_barrier(void* const* flags, int world, int rank, uint32_t epoch, int64_t limit_us,
                     int32_t* status, void* stream);

/* The other half of the exchange, one kernel per rank: for the rows this rank owns,
 * out = bf16(h + sum over ranks of slots[w]) (fp32, ranks in index order), written into every
 * rank's output buffer (outs: host array of `world` device pointers to contiguous (M, cols)
 * buffers, peer-mapped).  slots: this rank's (world, rows_per_owner, cols) receive region;
 * h: the local (M, cols) residual with leading dimension ld_h.  cols % 8 == 0. */
int lcg_reduce_gather(const void* slots, const void* h, int64_t ld_h, void* const* outs,
                      int64_t M, int64_t cols, int64_t rows_per_owner, int world, int rank,
                      void* stream);

/* Rank-7 C = A @ B^T straight from the activation matrix, for callers that cannot
 * allocate device memory.  This entry point has no counterpart in the reference.
 *
 * Who needs it: hosts that give all free device memory to their own pool at start-up
 * (an inference server sizing its KV cache from what is left), so that a plugin's
 * later cudaMalloc fails or eats into that pool, and serving paths on which
 * allocation is forbidden because cudaMalloc synchronises the device.
 *
 * The A planes -- the scratch lcg_a_planes + lcg_gemm_r7 keep in a caller-owned buffer
 * -- live in a fixed array of lcg_static_scratch_bytes() (32 MiB) of device memory
 * inside the library.  A GPU takes that memory when the array's address is first
 * resolved on it -- by lcg_static_reserve() or by the first lcg_gemm_r7_static call
 * there (CUDA loads modules lazily) -- and holds it until the process exits; that first
 * resolution may fail for lack of memory or synchronise the device, so a host that sizes
 * its pool from the free memory, or that must not stall later, calls
 * lcg_static_reserve() on every device at start-up, before it sizes the pool (or runs
 * with CUDA_MODULE_LOADING=EAGER).  After that the call allocates and frees nothing.
 * Limits and rules:
 *   - rank * ceil(M/2) * round_up(ceil(K/2), 64) * 2 bytes must fit in the array
 *     (e.g. M = 2048, K = 4096); larger shapes return LCG_ERR_UNSUPPORTED_SHAPE;
 *   - the first call on a device resolves the array's address (once per device, with
 *     that device current); make that first call before any stream capture begins;
 *   - all calls on a device share the one array: calls that overlap on the GPU
 *     (different streams) race.  Nothing needs clearing between calls -- each call
 *     rewrites every plane element it reads, padding included;
 *   - as for lcg_gemm_r7: a (M, K) with lda, B planes from lcg_prepare_b, ldc a
 *     multiple of 8, and C zeroed by the caller for LCG_SCHEDULE_RANK_SPLIT. */
int lcg_gemm_r7_static(const lcg_scheme_t* scheme, const void* a, int64_t lda,
                       const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                       int64_t M, int64_t N, int64_t K, int schedule, int cta_group,
                       int32_t* status, void* stream);
int64_t lcg_static_scratch_bytes(void);
/* Resolve the static scratch of the current device now (takes its memory there; see above).
 * Idempotent.  No counterpart in the reference. */
int lcg_static_reserve(void);

/* ---- dense-arm seams (the stock layer the rank-7 path is compared with) -- */

/* h = bf16(delta + residual) -> residual_out; x = bf16(rmsnorm(h) * (w + 1))
 * (lcgemm/integrate/qwen_patch.py:49-52). Contiguous (M, K), K % 8 == 0.
 * delta may be NULL as for lcg_norm_planes: h is the residual, residual_out is not written. */
int lcg_add_rmsnorm(const void* delta, const void* residual, const void* norm_weight,
                    int64_t M, int64_t K, float eps, void* residual_out, void* x,
                    void* stream);

/* s = bf16(silu(float(gate))) * up  (lcgemm/integrate/qwen_patch.py:54-56).
 * z is (M, 2*I) with ldz; s is (M, I) with lds. I % 8 == 0. */
int lcg_swiglu(const void* z, int64_t M, int64_t I, int64_t ldz, void* s, int64_t lds,
               void* stream);

/* out = bf16(float(a) + float(b)), n elements (the residual add that closes
 * the layer in config form `x + mlp(x)`). n % 8 == 0. */
int lcg_add(const void* a, const void* b, void* out, int64_t n, void* stream);

/* ---- introspection ------------------------------------------------------- */

/* Kernel launches issued by this library in this process (for the bench's
 * `gpu_launches`). */
int64_t lcg_launch_count(void);

/* Exercise the bounded device-side wait: a one-CTA kernel waits (for at most limit_us
 * microseconds) on a barrier nothing signals, so the wait runs out, writes code 199 into
 * `status` and the kernel returns; `finished` (device int32, may be NULL) receives 1.  Shows
 * a host how a stuck pipeline surfaces: as a status code, never as a hung context. */
int lcg_selftest_wait_timeout(int32_t* status, int64_t limit_us, int32_t* finished, void* stream);

/* One line describing the schedule the GEMM entry points would pick for a
 * shape (tile, stages, units, CTA groups); the counterpart of the reference's
 * Plan.describe() (lcgemm/kernels/sm100.py:358-374). Returns bytes written. */
int lcg_describe_gemm(int64_t M, int64_t N, int64_t K, int rank7, int schedule,
                      int cta_group, char* buf, int buflen);

#ifdef __cplusplus
}
#endif
#endif /* LCGEMM_B200_H */
