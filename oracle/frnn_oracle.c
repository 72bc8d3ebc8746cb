/*
 * CPU oracle for the FlashRNN recurrent hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference's `vanilla` backend
 * (the PyTorch loop every reference test compares against) together with the closed-form
 * per-step backward that the reference's CUDA and hand-written PyTorch paths use.  Nothing in
 * the shipped CUDA product path may call into it: only the tests, the smoke check and the
 * benchmark's CPU-baseline leg load this library, and only as the checker.
 *
 * Parity pin: the functions below are checked against golden vectors produced by importing the
 * unmodified reference (`flashrnn(..., backend="vanilla")`, fp64 and fp32, forward and autograd
 * backward) -- see tests/golden/make_golden.py and tests/test_oracle_golden.py.
 *
 * Reference lines followed (paths inside the reference project):
 *   time loop, Ry = h . R^T per head ............ flashrnn/flashrnn/vanilla/__init__.py:20-70
 *   LSTM cell ................................... flashrnn/flashrnn/vanilla/lstm.py:4-31
 *   GRU cell .................................... flashrnn/flashrnn/vanilla/gru.py:4-32
 *   Elman cell .................................. flashrnn/flashrnn/vanilla/elman.py:4-23
 *   sLSTM cell .................................. flashrnn/flashrnn/vanilla/slstm.py:4-35
 *   user layouts Wx[B,T,G,N,D] R[G,N,D,D] b[G,N,D]  flashrnn/flashrnn/flashrnn.py:165-173, 1114-1135
 *   LSTM / sLSTM closed-form backward ........... flashrnn/flashrnn/vanilla_fwbw/bw.py:100-189
 *   GRU closed-form backward .................... flashrnn/flashrnn/alternating/gru_pointwise.cu:120-193
 *   Elman closed-form backward .................. flashrnn/flashrnn/fused/elman_fused_pointwise.cuh:62-93
 *   per-element "m' = i~ when n == 0" rule ...... flashrnn/flashrnn/fused/slstm_fused_pointwise.cuh:53-62
 *
 * The file is compiled twice (REAL=double -> *_f64 symbols, REAL=float -> *_f32 symbols).
 *
 * Layouts (all dense, row-major, exactly the reference's user-facing layouts):
 *   Wx      [B][T][Gw][N][D]     inputs (already projected)
 *   R       [Gr][N][D][D]        R[g][n][d_out][d_in]
 *   b       [Gt][N][D]
 *   s0      [S][B][N][D]         initial states (the reference's [S,B,1,N,D] with the 1 squeezed)
 *   states  [S][B][T][N][D]      state s after step t
 *   cache   [B][T][GC][N][D]     values the closed-form backward needs (GC = 5 for every cell here)
 *   dstates [S][B][T][N][D]      cotangent of `states`
 *   dWx like Wx, dR like R, db like b, ds0 like s0
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL double
#endif
#ifndef SUFFIX
#define SUFFIX f64
#endif
#define CAT_(a, b) a##_##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

#if defined(__x86_64__) && defined(__GNUC__) && !defined(FRNN_ORACLE_NO_CLONES)
#define HOT __attribute__((target_clones("avx2,fma", "default")))
#else
#define HOT
#endif

enum { CELL_LSTM = 0, CELL_GRU = 1, CELL_ELMAN = 2, CELL_SLSTM = 3 };
enum { GC = 5 }; /* cache slots per (b,t,n,d) */

/* gate / state counts per cell: reference flashrnn.py:49-71 (Gr, Gw, Gi, Gt, S) */
static int cell_dims(int cell, int* Gr, int* Gw, int* Gt, int* S) {
  switch (cell) {
    case CELL_LSTM:  *Gr = 4; *Gw = 4; *Gt = 4; *S = 2; return 0;
    case CELL_GRU:   *Gr = 3; *Gw = 3; *Gt = 4; *S = 1; return 0;
    case CELL_ELMAN: *Gr = 1; *Gw = 1; *Gt = 1; *S = 1; return 0;
    case CELL_SLSTM: *Gr = 4; *Gw = 4; *Gt = 4; *S = 4; return 0;
  }
  return -1;
}

static inline REAL sigm(REAL x) { return (REAL)1 / ((REAL)1 + (REAL)exp(-(double)x)); }
static inline REAL logsigm(REAL x) {
  /* log(sigmoid(x)) = min(x,0) - log1p(exp(-|x|)) */
  double ax = fabs((double)x);
  return (REAL)(((double)x < 0 ? (double)x : 0.0) - log1p(exp(-ax)));
}

/* pre[g][d] = sum_p R[g][n][d][p] * h[p]   (vanilla/__init__.py:53-61) */
HOT static void recurrent_matvec(const REAL* restrict R, int Gr, int N, int D, int n, const REAL* restrict h,
                                 REAL* restrict pre) {
  for (int g = 0; g < Gr; ++g) {
    const REAL* Rg = R + (((size_t)g * N + n) * D) * D;
    for (int d = 0; d < D; ++d) {
      const REAL* row = Rg + (size_t)d * D;
      REAL acc = 0;
      /* the sum may be formed in vector lanes (a different association than left to right: rounding-level effect) */
#pragma omp simd reduction(+ : acc)
      for (int p = 0; p < D; ++p) acc += row[p] * h[p];
      pre[g * D + d] = acc;
    }
  }
}

/* dh[p] += sum_{g,d} delta[g][d] * R[g][n][d][p] ;  dRn[g][d][p] += delta[g][d] * hprev[p] */
HOT static void recurrent_backward(const REAL* restrict R, int Gr, int N, int D, int n, const REAL* restrict delta,
                                   const REAL* restrict hprev, REAL* restrict dh, REAL* restrict dRn) {
  for (int g = 0; g < Gr; ++g) {
    const REAL* Rg = R + (((size_t)g * N + n) * D) * D;
    REAL* dRg = dRn + (size_t)g * D * D;
    for (int d = 0; d < D; ++d) {
      const REAL dl = delta[g * D + d];
      const REAL* row = Rg + (size_t)d * D;
      REAL* drow = dRg + (size_t)d * D;
#pragma omp simd
      for (int p = 0; p < D; ++p) {
        dh[p] += dl * row[p];
        drow[p] += dl * hprev[p];
      }
    }
  }
}

/*
 * Forward.  `slstm_global_rule` != 0 selects the vanilla backend's rule "m' = i~ iff ALL entries of n
 * (whole [B,N,D] tensor) are zero" (vanilla/slstm.py:21-24); 0 selects the per-element rule of the
 * reference's CUDA kernels.  For all-zero initial states the two agree.
 * `fclip` > 0 clamps every new h to [-fclip, fclip] (the reference's forward_clipval,
 * flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:75-80).  `cache` may be NULL (inference).  Returns 0, or -1 on a bad cell id / allocation failure.
 */
int FN(frnn_oracle_forward)(int cell, int B, int T, int N, int D, const REAL* Wx, const REAL* R, const REAL* b,
                            const REAL* s0, REAL* states, REAL* cache, int slstm_global_rule, double fclip) {
  int Gr, Gw, Gt, S;
  if (cell_dims(cell, &Gr, &Gw, &Gt, &S)) return -1;
  const size_t ND = (size_t)N * D;

  /* vanilla sLSTM tests n == 0 over the whole tensor each step.  Rows evolve independently, so the
   * global flag at step t is "every (b,n,d) still has n == 0", which after step 0 is never true
   * (n' >= 1).  Hence: step 0 uses the global test on the initial n, later steps use max(). */
  int all_n0_zero = 1;
  if (cell == CELL_SLSTM) {
    const REAL* n0 = s0 + (size_t)2 * B * ND;
    for (size_t i = 0; i < (size_t)B * ND; ++i)
      if (n0[i] != (REAL)0) { all_n0_zero = 0; break; }
  }
  int fail = 0;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int bb = 0; bb < B; ++bb) {
    for (int n = 0; n < N; ++n) {
      REAL* pre = (REAL*)malloc(sizeof(REAL) * (size_t)(Gr + 4) * D);
      if (!pre) { fail = 1; continue; }
      REAL* st = pre + (size_t)Gr * D; /* running states [S][D], S <= 4 */
      for (int s = 0; s < S; ++s)
        memcpy(st + (size_t)s * D, s0 + ((size_t)s * B + bb) * ND + (size_t)n * D, sizeof(REAL) * D);
      for (int t = 0; t < T; ++t) {
        recurrent_matvec(R, Gr, N, D, n, st, pre);
        const REAL* wx = Wx + (((size_t)bb * T + t) * Gw) * ND + (size_t)n * D; /* + g*ND + d */
        REAL* ch = cache ? cache + (((size_t)bb * T + t) * GC) * ND + (size_t)n * D : NULL;
        for (int d = 0; d < D; ++d) {
#define BIAS(g) b[((size_t)(g) * N + n) * D + d]
#define WX(g) wx[(size_t)(g) * ND + d]
#define PRE(g) pre[(g) * D + d]
#define CACHE(k) ch[(size_t)(k) * ND + d]
          if (cell == CELL_LSTM) {
            REAL ig = sigm(WX(0) + PRE(0) + BIAS(0));
            REAL fg = sigm(WX(1) + PRE(1) + BIAS(1));
            REAL zv = (REAL)tanh((double)(WX(2) + PRE(2) + BIAS(2)));
            REAL og = sigm(WX(3) + PRE(3) + BIAS(3));
            REAL cn = fg * st[D + d] + ig * zv;
            REAL hn = og * (REAL)tanh((double)cn);
            if (ch) { CACHE(0) = ig; CACHE(1) = fg; CACHE(2) = zv; CACHE(3) = og; CACHE(4) = 0; }
            st[d] = hn; st[D + d] = cn;
          } else if (cell == CELL_GRU) {
            REAL gr = PRE(0) + BIAS(0);
            REAL rg = sigm(WX(0) + PRE(1) + BIAS(1));
            REAL zg = sigm(WX(1) + PRE(2) + BIAS(2));
            REAL nr = WX(2) + BIAS(3);
            REAL nv = (REAL)tanh((double)(nr + rg * gr));
            REAL hn = zg * st[d] + ((REAL)1 - zg) * nv;
            if (ch) { CACHE(0) = gr; CACHE(1) = rg; CACHE(2) = zg; CACHE(3) = nv; CACHE(4) = 0; }
            st[d] = hn;
          } else if (cell == CELL_ELMAN) {
            REAL hn = (REAL)tanh((double)(WX(0) + PRE(0) + BIAS(0)));
            if (ch) { CACHE(0) = hn; CACHE(1) = 0; CACHE(2) = 0; CACHE(3) = 0; CACHE(4) = 0; }
            st[d] = hn;
          } else { /* sLSTM */
            REAL ir = WX(0) + PRE(0) + BIAS(0);
            REAL fr = WX(1) + PRE(1) + BIAS(1);
            REAL zv = (REAL)tanh((double)(WX(2) + PRE(2) + BIAS(2)));
            REAL og = sigm(WX(3) + PRE(3) + BIAS(3));
            REAL c = st[D + d], nn = st[2 * D + d], m = st[3 * D + d];
            REAL lfm = logsigm(fr) + m;
            int first = slstm_global_rule ? (t == 0 && all_n0_zero) : (nn == (REAL)0);
            REAL mn = first ? ir : (ir > lfm ? ir : lfm);
            REAL ig = (REAL)exp((double)(ir - mn));
            REAL fg = (REAL)exp((double)(lfm - mn));
            REAL cn = fg * c + ig * zv;
            REAL n2 = fg * nn + ig;
            if (n2 < (REAL)1) n2 = (REAL)1;
            REAL hn = og * cn / n2;
            if (ch) { CACHE(0) = ig; CACHE(1) = fg; CACHE(2) = zv; CACHE(3) = og; CACHE(4) = (REAL)1 - sigm(fr); }
            st[d] = hn; st[D + d] = cn; st[2 * D + d] = n2; st[3 * D + d] = mn;
          }
        }
        if (fclip > 0)
          for (int d = 0; d < D; ++d) {
            if (st[d] > (REAL)fclip) st[d] = (REAL)fclip;
            if (st[d] < (REAL)-fclip) st[d] = (REAL)-fclip;
          }
        for (int s = 0; s < S; ++s)
          memcpy(states + (((size_t)s * B + bb) * T + t) * ND + (size_t)n * D, st + (size_t)s * D, sizeof(REAL) * D);
      }
      free(pre);
    }
  }
  return fail ? -1 : 0;
}

/*
 * Closed-form backward through time.  Needs `states` and `cache` from the forward above.
 * The sLSTM stabiliser m is treated as a constant (as in the reference's CUDA and manual-PyTorch
 * backward); this equals full autograd for cotangents that reach the loss through h only.
 * `clip` > 0 clamps the recurrent part of dh to [-clip, clip] before use (gradient_recurrent_clipval).
 * `cut` != 0 drops the R^T delta term of dh_{t-1} (the reference's gradient_recurrent_cut,
 * flashrnn/flashrnn/fused/flashrnn_fused_backward_cut.cu:89-178); dR is still formed from the deltas.
 * dR, db are overwritten (not accumulated into).
 */
int FN(frnn_oracle_backward)(int cell, int B, int T, int N, int D, const REAL* R, const REAL* s0, const REAL* states,
                             const REAL* cache, const REAL* dstates, REAL* dWx, REAL* dR, REAL* db, REAL* ds0,
                             double clip, int cut) {
  int Gr, Gw, Gt, S;
  if (cell_dims(cell, &Gr, &Gw, &Gt, &S)) return -1;
  const size_t ND = (size_t)N * D;
  memset(dR, 0, sizeof(REAL) * (size_t)Gr * N * D * D);
  memset(db, 0, sizeof(REAL) * (size_t)Gt * ND);
  int fail = 0;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int n = 0; n < N; ++n) {
    for (int bb = 0; bb < B; ++bb) {
      const size_t nDD = (size_t)Gr * D * D;
      REAL* dRn = (REAL*)calloc(nDD + (size_t)(4 + 4 + 4 + 2) * D, sizeof(REAL));
      if (!dRn) { fail = 1; continue; }
      REAL* dbn = dRn + nDD;           /* [4][D]  bias-gate sums    */
      REAL* delta = dbn + (size_t)4 * D; /* [Gr][D] R-gate deltas     */
      REAL* carry = delta + (size_t)4 * D; /* [4][D] recurrent cotangent of each state */
      REAL* dhn = carry + (size_t)4 * D; /* [D]    R^T delta (next carry of h) */
      REAL* hprev = dhn + D;
      for (int t = T - 1; t >= 0; --t) {
        const REAL* ch = cache + (((size_t)bb * T + t) * GC) * ND + (size_t)n * D;
        REAL* dwx = dWx + (((size_t)bb * T + t) * Gw) * ND + (size_t)n * D;
#define ST(s, tt) states[(((size_t)(s) * B + bb) * T + (tt)) * ND + (size_t)n * D + d]
#define S0(s) s0[((size_t)(s) * B + bb) * ND + (size_t)n * D + d]
#define PREV(s) (t > 0 ? ST(s, t - 1) : S0(s))
#define DEXT(s) dstates[(((size_t)(s) * B + bb) * T + t) * ND + (size_t)n * D + d]
        for (int d = 0; d < D; ++d) {
          REAL rec = carry[d];
          if (clip > 0) { if (rec > (REAL)clip) rec = (REAL)clip; if (rec < (REAL)-clip) rec = (REAL)-clip; }
          REAL dh = DEXT(0) + rec;
          hprev[d] = PREV(0);
          if (cell == CELL_LSTM) {
            REAL ig = CACHE(0), fg = CACHE(1), zv = CACHE(2), og = CACHE(3);
            REAL tc = (REAL)tanh((double)ST(1, t));
            REAL dc = DEXT(1) + carry[D + d] + dh * og * ((REAL)1 - tc * tc);
            REAL di = dc * zv * ig * ((REAL)1 - ig);
            REAL df = dc * PREV(1) * fg * ((REAL)1 - fg);
            REAL dz = dc * ig * ((REAL)1 - zv * zv);
            REAL dO = dh * tc * og * ((REAL)1 - og);
            delta[d] = di; delta[D + d] = df; delta[2 * D + d] = dz; delta[3 * D + d] = dO;
            dwx[d] = di; dwx[ND + d] = df; dwx[2 * ND + d] = dz; dwx[3 * ND + d] = dO;
            dbn[d] += di; dbn[D + d] += df; dbn[2 * D + d] += dz; dbn[3 * D + d] += dO;
            carry[d] = 0; carry[D + d] = dc * fg;
          } else if (cell == CELL_GRU) {
            REAL gr = CACHE(0), rg = CACHE(1), zg = CACHE(2), nv = CACHE(3);
            REAL dz = dh * (hprev[d] - nv) * zg * ((REAL)1 - zg);
            REAL dn = dh * ((REAL)1 - zg) * ((REAL)1 - nv * nv);
            REAL dr = dn * gr * rg * ((REAL)1 - rg);
            REAL dg = dn * rg;
            delta[d] = dg; delta[D + d] = dr; delta[2 * D + d] = dz;
            dwx[d] = dr; dwx[ND + d] = dz; dwx[2 * ND + d] = dn;
            dbn[d] += dg; dbn[D + d] += dr; dbn[2 * D + d] += dz; dbn[3 * D + d] += dn;
            carry[d] = zg * dh;
          } else if (cell == CELL_ELMAN) {
            REAL hn = CACHE(0);
            REAL dg = dh * ((REAL)1 - hn * hn);
            delta[d] = dg; dwx[d] = dg; dbn[d] += dg;
            carry[d] = 0;
          } else { /* sLSTM, bw.py:136-189 */
            REAL ig = CACHE(0), fg = CACHE(1), zv = CACHE(2), og = CACHE(3), omsf = CACHE(4);
            REAL cn = ST(1, t), n2 = ST(2, t);
            REAL dc = DEXT(1) + carry[D + d] + dh * og / n2;
            REAL dn = DEXT(2) + carry[2 * D + d] - dh * og * cn / (n2 * n2);
            REAL di = ig * (zv * dc + dn);
            REAL df = fg * (dc * PREV(1) + dn * PREV(2)) * omsf;
            REAL dz = dc * ig * ((REAL)1 - zv * zv);
            REAL dO = dh * (cn / n2) * og * ((REAL)1 - og);
            delta[d] = di; delta[D + d] = df; delta[2 * D + d] = dz; delta[3 * D + d] = dO;
            dwx[d] = di; dwx[ND + d] = df; dwx[2 * ND + d] = dz; dwx[3 * ND + d] = dO;
            dbn[d] += di; dbn[D + d] += df; dbn[2 * D + d] += dz; dbn[3 * D + d] += dO;
            carry[d] = 0; carry[D + d] = fg * dc; carry[2 * D + d] = fg * dn; carry[3 * D + d] = 0;
          }
        }
        memset(dhn, 0, sizeof(REAL) * D);
        recurrent_backward(R, Gr, N, D, n, delta, hprev, dhn, dRn);
        if (!cut)
          for (int d = 0; d < D; ++d) carry[d] += dhn[d];
      }
      for (int s = 0; s < S; ++s)
        for (int d = 0; d < D; ++d) ds0[((size_t)s * B + bb) * ND + (size_t)n * D + d] = carry[(size_t)s * D + d];
#pragma omp critical
      {
        for (int g = 0; g < Gr; ++g) {
          REAL* dst = dR + (((size_t)g * N + n) * D) * D;
          const REAL* src = dRn + (size_t)g * D * D;
          for (size_t i = 0; i < (size_t)D * D; ++i) dst[i] += src[i];
        }
        for (int g = 0; g < Gt; ++g)
          for (int d = 0; d < D; ++d) db[((size_t)g * N + n) * D + d] += dbn[(size_t)g * D + d];
      }
      free(dRn);
    }
  }
  return fail ? -1 : 0;
}

int FN(frnn_oracle_cache_slots)(void) { return GC; }
