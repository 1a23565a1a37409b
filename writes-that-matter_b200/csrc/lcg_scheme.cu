// Native side of the scheme layer: validates a 2x2x2 rank-R decomposition in
// exact integer arithmetic and derives the per-step epilogue plan the GEMM
// kernel walks.  Mirrors the behaviour of the reference's host-side Scheme
// (lcgemm/scheme.py:204-264 chains / sigma / groups, :324-408 validation);
// the host-side Python Scheme derives the same tables independently and the
// tests cross-check the two through lcg_scheme_plan().
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <new>

#include "lcg_common.h"

namespace lcg {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

struct Pub {  // one publication: coeff * (accumulator) -> C block (bi, bj)
  int bi, bj, coeff;
};

// Group one step's publications by coefficient, positive coefficients first,
// and mark the lowest contributing step of each block as its first writer.
int build_step(const Pub* pubs, int npubs, const int first_writer[2][2], int step,
               bool store_first, StepDesc* out) {
  int coeffs[4];
  int ncoef = 0;
  for (int n = 0; n < npubs; ++n) {
    bool seen = false;
    for (int m = 0; m < ncoef; ++m) seen = seen || coeffs[m] == pubs[n].coeff;
    if (!seen) coeffs[ncoef++] = pubs[n].coeff;
  }
  std::sort(coeffs, coeffs + ncoef, [](int x, int y) { return x > y; });
  if (ncoef > 2)
    return fail(LCG_ERR_SCHEME, "step %d publishes with %d distinct coefficients; at most 2 supported",
                step, ncoef);
  out->ngroups = ncoef;
  for (int g = 0; g < ncoef; ++g) {
    EpiGroup& grp = out->group[g];
    grp.coeff = coeffs[g];
    grp.ndest = 0;
    for (int n = 0; n < npubs; ++n) {
      if (pubs[n].coeff != coeffs[g]) continue;
      EpiDest& d = grp.dest[grp.ndest++];
      d.bi = static_cast<int8_t>(pubs[n].bi);
      d.bj = static_cast<int8_t>(pubs[n].bj);
      d.first = static_cast<int8_t>(store_first && first_writer[pubs[n].bi][pubs[n].bj] == step);
      d.pad = 0;
    }
  }
  return LCG_OK;
}

int validate_identity(const lcg_scheme& s) {
  // sum_r c[r][i,j] a[r][i',k'] b[r][k'',j''] must be 1 exactly on
  // (i'=i, k'=k'', j''=j) and 0 elsewhere.
  for (int i = 0; i < 2; ++i)
    for (int j = 0; j < 2; ++j)
      for (int ip = 0; ip < 2; ++ip)
        for (int kp = 0; kp < 2; ++kp)
          for (int kpp = 0; kpp < 2; ++kpp)
            for (int jpp = 0; jpp < 2; ++jpp) {
              int acc = 0;
              for (int r = 0; r < s.rank; ++r)
                acc += s.c[r][i * 2 + j] * s.a[r][ip * 2 + kp] * s.b[r][kpp * 2 + jpp];
              const int want = (ip == i && kp == kpp && jpp == j) ? 1 : 0;
              if (acc != want)
                return fail(LCG_ERR_SCHEME,
                            "not a decomposition of the block product: A[%d][%d]*B[%d][%d] reaches "
                            "C[%d][%d] with coefficient %d, expected %d",
                            ip, kp, kpp, jpp, i, j, acc, want);
            }
  return LCG_OK;
}

}  // namespace
}  // namespace lcg

using namespace lcg;

extern "C" int lcg_version(void) { return 100; }

extern "C" const char* lcg_last_error(void) { return g_error; }

extern "C" int64_t lcg_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int lcg_scheme_create(const int8_t* a, const int8_t* b, const int8_t* c, int rank,
                                 const int8_t* clear, lcg_scheme_t** out) {
  if (out == nullptr) return fail(LCG_ERR_BAD_ARG, "out is NULL");
  *out = nullptr;
  if (a == nullptr || b == nullptr || c == nullptr)
    return fail(LCG_ERR_BAD_ARG, "coefficient tables must not be NULL");
  if (rank < 1 || rank > kMaxRank)
    return fail(LCG_ERR_SCHEME, "rank %d outside [1, %d]", rank, kMaxRank);

  lcg_scheme s;
  std::memset(&s, 0, sizeof(s));
  s.rank = rank;
  s.has_postsum = clear != nullptr;
  for (int r = 0; r < rank; ++r) {
    bool za = true, zb = true, zc = true;
    for (int x = 0; x < 4; ++x) {
      s.a[r][x] = a[r * 4 + x];
      s.b[r][x] = b[r * 4 + x];
      s.c[r][x] = c[r * 4 + x];
      za = za && s.a[r][x] == 0;
      zb = zb && s.b[r][x] == 0;
      zc = zc && s.c[r][x] == 0;
    }
    if (za || zb || zc)
      return fail(LCG_ERR_SCHEME, "product %d has an all-zero coefficient row", r);
    if (clear != nullptr && clear[r] != 0 && clear[r] != 1)
      return fail(LCG_ERR_SCHEME, "clear[%d] = %d is not 0/1", r, clear[r]);
    s.clear[r] = clear != nullptr ? clear[r] : 1;
  }
  if (int e = validate_identity(s)) return e;
  for (int t = 0; t < std::min(2, rank); ++t)
    if (!s.clear[t])
      return fail(LCG_ERR_SCHEME, "step %d continues an accumulator chain that never started", t);

  // Chains: step t owns accumulator stage t % 2; a chain is the run of
  // same-parity steps after a clear.  next[t] = following step of t's chain.
  int next[kMaxRank];
  int open[2] = {-1, -1};
  for (int t = 0; t < rank; ++t) {
    next[t] = -1;
    const int stage = t & 1;
    if (!s.clear[t] && open[stage] >= 0) next[open[stage]] = t;
    open[stage] = t;
  }
  // sigma_t = c[t] - c[next(t)]: what publishing the prefix sum at step t must
  // carry so that the prefixes telescope back to C.
  Pub pubs[kMaxRank][4];
  int npubs[kMaxRank];
  int first_writer[2][2] = {{-1, -1}, {-1, -1}};
  for (int t = 0; t < rank; ++t) {
    npubs[t] = 0;
    for (int x = 0; x < 4; ++x) {
      const int sigma = s.c[t][x] - (next[t] >= 0 ? s.c[next[t]][x] : 0);
      if (sigma == 0) continue;
      pubs[t][npubs[t]++] = Pub{x / 2, x % 2, sigma};
      if (first_writer[x / 2][x % 2] < 0) first_writer[x / 2][x % 2] = t;
    }
  }
  // Telescoping check: the coefficient product u ends up with in block x is
  // the sum of sigma over u's chain from u onwards.
  for (int u = 0; u < rank; ++u)
    for (int x = 0; x < 4; ++x) {
      int got = 0;
      for (int t = u; t >= 0; t = next[t]) {
        for (int n = 0; n < npubs[t]; ++n)
          if (pubs[t][n].bi * 2 + pubs[t][n].bj == x) got += pubs[t][n].coeff;
      }
      if (got != s.c[u][x])
        return fail(LCG_ERR_SCHEME, "chain plan does not reproduce C for product %d block %d", u, x);
    }
  for (int x = 0; x < 4; ++x)
    if (first_writer[x / 2][x % 2] < 0)
      return fail(LCG_ERR_SCHEME, "C block (%d,%d) is never written", x / 2, x % 2);

  for (int t = 0; t < rank; ++t) {
    StepDesc& st = s.all_ranks[t];
    st.a_plane = t;
    st.b_plane = t;
    st.clear = s.clear[t];
    if (int e = build_step(pubs[t], npubs[t], first_writer, t, true, &st)) return e;

    // Rank split: product t alone, scattered by reduce-add over its C row.
    Pub own[4];
    int nown = 0;
    for (int x = 0; x < 4; ++x)
      if (s.c[t][x]) own[nown++] = Pub{x / 2, x % 2, s.c[t][x]};
    StepDesc& rs = s.rank_split[t];
    rs.a_plane = t;
    rs.b_plane = t;
    rs.clear = 1;
    if (int e = build_step(own, nown, first_writer, t, false, &rs)) return e;
  }

  lcg_scheme* heap = new (std::nothrow) lcg_scheme(s);
  if (heap == nullptr) return fail(LCG_ERR_BAD_ARG, "out of host memory");
  *out = heap;
  return LCG_OK;
}

extern "C" void lcg_scheme_destroy(lcg_scheme_t* scheme) { delete scheme; }

extern "C" int lcg_scheme_plan(const lcg_scheme_t* scheme, int8_t* out, int32_t* counts) {
  if (scheme == nullptr || out == nullptr || counts == nullptr)
    return fail(LCG_ERR_BAD_ARG, "NULL argument");
  for (int t = 0; t < scheme->rank; ++t) {
    int n = 0;
    const StepDesc& st = scheme->all_ranks[t];
    for (int g = 0; g < st.ngroups; ++g)
      for (int d = 0; d < st.group[g].ndest; ++d) {
        int8_t* rec = out + t * 16 + 4 * n++;
        rec[0] = st.group[g].dest[d].bi;
        rec[1] = st.group[g].dest[d].bj;
        rec[2] = static_cast<int8_t>(st.group[g].coeff);
        rec[3] = st.group[g].dest[d].first;
      }
    counts[t] = n;
  }
  return LCG_OK;
}

extern "C" int lcg_plane_geometry(int64_t rows, int64_t cols, int row_align, int64_t* rows2,
                                  int64_t* k2, int64_t* k2p) {
  if (rows < 1 || cols < 1 || row_align < 1) return fail(LCG_ERR_BAD_ARG, "bad extents");
  const int64_t r2 = (rows + 1) / 2;
  const int64_t kk = (cols + 1) / 2;
  if (rows2) *rows2 = (r2 + row_align - 1) / row_align * row_align;
  if (k2) *k2 = kk;
  if (k2p) *k2p = (kk + 63) / 64 * 64;
  return LCG_OK;
}
