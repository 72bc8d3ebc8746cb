// float32 kernel dtype: Wx, R, b, the states and every gradient are fp32 and so is all arithmetic.
//
// The reference offers dtype="float32" for every cell (tests/test_lstm.py:48-60; its fused kernel then multiplies in
// tf32, fused/flashrnn_fused_forward.cu:108-112).  Here the fp32 path is the ACCURATE one: products and sums in fp32 on
// the CUDA cores, gate nonlinearities from exp (error ~1e-6), so that it agrees with the fp32 `vanilla` loop to ~1e-5 --
// the 16-bit tensor-core loops are the fast path, this one is for callers that need float32 results (reference checks,
// gradient checks, small models).
//   * cluster loops (x32c_*): a cluster of CS CTAs owns one head and 8 batch rows for all T steps; CTA c owns U = D / CS
//     units, keeps its slice of R in shared memory as fp32 (Gr*U*D*4 bytes) and exchanges per step only what the others
//     need -- its slice of h_t (forward, all-gather) or its partial sums of dh_{t-1} (reverse, reduce-scatter) -- with
//     one bulk copy per peer that completes on the peer's mbarrier, the protocol of the 16-bit loops.  A thread's items
//     (batch row, unit) are fixed, so states, carried cotangents and bias stay in registers and the next step's global
//     inputs are loaded one step ahead.  The matrix phase is FFMA from shared memory: a thread keeps 16 (forward: two
//     gate rows x 8 batch rows) or 8 (reverse: one column x 8 batch rows) sums over its share of k.
//   * streamed loops (x32_*): one CTA per (head, 8 batch rows), R read from L2 in every step; for head dims whose slices
//     do not fit the shared memory of a portable cluster (e.g. four-gate cells above 256) or are no multiple of 4 units.
//   * dR: a tiled fp32 GEMM over all (b, t) with split-K and fp32 atomics.
// Replaces, for float32, FLASHRNNCellFusedForward / FLASHRNNCellFusedBackward / the cuBLAS dR GEMM of the reference
// (fused/flashrnn_fused_forward.cu:146-659, fused/flashrnn_fused_backward.cu:129-624, 1049-1058).
#ifndef FRNN_F16  // compiled once, into the bfloat16 build, which owns the public entry points
#define FRNN_NS_OVERRIDE frnn_x32
#define FRNN_EXACT_ACT 1
#include <type_traits>

#include "../../include/frnn.h"
#include "frnn_bwd.cuh"
#include "frnn_fwd.cuh"

namespace FRNN_NS {

namespace {

constexpr int XBT = 8;        // batch rows per CTA
constexpr int XTHREADS = 256;
constexpr size_t kStatus = 256;
constexpr size_t kSmemMax = 227 * 1024;

struct XParams {
  const float* Wx; const float* R; const float* RT; const float* bias; const float* s0;
  float* states; float* cache;
  const float* dstates; float* dWx; float* dg0; float* ds0; float* dbias;
  unsigned* status;
  int B, T, N, D;
  int U, CS, KS;  // cluster loops: units per CTA, CTAs per cluster, k-splits of the matrix phase
  int test_drop;  // test hook: CTA 0 of every cluster withholds its message of step 1
  int r_in_smem;
  float fclip, gclip;
  int grad_cut;
  long long wx_sb, wx_st, wx_sg, wx_sn, ds_ss, ds_sb, ds_st, ds_sn;
};

// RT[n][p][g*D + d] = R[g][n][d][p]
__global__ void transpose_recurrent_kernel(const float* __restrict__ R, float* __restrict__ RT, int Gr, int N, int D) {
  const size_t total = (size_t)Gr * N * D * D;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int gd = (int)(i % ((size_t)Gr * D));
  size_t r = i / ((size_t)Gr * D);
  const int p = (int)(r % D);
  const int n = (int)(r / D);
  const int g = gd / D, d = gd - g * D;
  RT[i] = R[(((size_t)g * N + n) * D + d) * D + p];
}

// acc[b] (b < 8) += sum_k w[k * wstride + col] * x[b * xstride + k], k < K: one output column `col` for the 8 batch rows
__device__ __forceinline__ void col_dot8(const float* __restrict__ w, size_t wstride, int col, const float* x, int xstride, int K,
                                         float (&acc)[XBT]) {
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const float wv = w[(size_t)k * wstride + col];
#pragma unroll
    for (int b = 0; b < XBT; ++b) acc[b] = fmaf(wv, x[b * xstride + k], acc[b]);
  }
}

template <int CELL>
__global__ void __launch_bounds__(XTHREADS) x32_fwd_kernel(const XParams p) {
  using C = Cell<CELL>;
  constexpr int Gr = C::Gr, Gw = C::Gw, Gt = C::Gt, S = C::S, GC = C::GC, GCA = GC > 0 ? GC : 1;
  extern __shared__ __align__(16) float sm[];
  const int D = p.D, N = p.N, T = p.T, B = p.B, GD = Gr * D;
  const int tid = threadIdx.x, n = blockIdx.y, b0 = blockIdx.x * XBT;
  const size_t ND = (size_t)N * D;
  float* h = sm;                   // [8][D]   h_{t-1}, rows beyond B stay zero
  float* pre = h + XBT * D;        // [8][GD]
  float* Rs = pre + XBT * GD;      // [D][GD]  (r_in_smem)
  const float* RT = p.RT + (size_t)n * D * GD;
  if (p.r_in_smem) {
    for (int i = tid; i < D * GD; i += XTHREADS) Rs[i] = RT[i];
    RT = Rs;
  }
  for (int i = tid; i < XBT * D; i += XTHREADS) {
    const int bl = i / D, d = i - bl * D, b = b0 + bl;
    h[i] = b < B ? p.s0[(size_t)b * ND + (size_t)n * D + d] : 0.f;
  }
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    for (int row = tid; row < GD; row += XTHREADS) {
      float acc[XBT];
#pragma unroll
      for (int b = 0; b < XBT; ++b) acc[b] = 0.f;
      col_dot8(RT, (size_t)GD, row, h, D, D, acc);
#pragma unroll
      for (int b = 0; b < XBT; ++b) pre[b * GD + row] = acc[b];
    }
    __syncthreads();
    for (int i = tid; i < XBT * D; i += XTHREADS) {
      const int bl = i / D, d = i - bl * D, b = b0 + bl;
      if (b >= B) continue;
      const size_t nd = (size_t)n * D + d;
      float prv[Gr], wx[Gw], bv[Gt], st[S], cv[GCA];
#pragma unroll
      for (int g = 0; g < Gr; ++g) prv[g] = pre[bl * GD + g * D + d];
#pragma unroll
      for (int g = 0; g < Gw; ++g) wx[g] = p.Wx[(size_t)b * p.wx_sb + (size_t)t * p.wx_st + (size_t)g * p.wx_sg + (size_t)n * p.wx_sn + d];
#pragma unroll
      for (int g = 0; g < Gt; ++g) bv[g] = p.bias[(size_t)g * ND + nd];
#pragma unroll
      for (int s = 0; s < S; ++s)
        st[s] = t > 0 ? p.states[(((size_t)s * B + b) * T + (t - 1)) * ND + nd] : p.s0[((size_t)s * B + b) * ND + nd];
      cell_forward<CELL>(prv, wx, bv, st, cv);
      if (p.fclip > 0.f) st[0] = clampf(st[0], p.fclip);
#pragma unroll
      for (int s = 0; s < S; ++s) p.states[(((size_t)s * B + b) * T + t) * ND + nd] = st[s];
      if (GC > 0 && p.cache != nullptr) {
#pragma unroll
        for (int k = 0; k < GC; ++k) p.cache[(((size_t)b * T + t) * GCA + k) * ND + nd] = cv[k];
      }
      h[i] = st[0];
    }
    __syncthreads();
  }
}

template <int CELL>
__global__ void __launch_bounds__(XTHREADS) x32_bwd_kernel(const XParams p) {
  using C = Cell<CELL>;
  constexpr int Gr = C::Gr, Gw = C::Gw, Gt = C::Gt, S = C::S, GC = C::GC, GCA = GC > 0 ? GC : 1, NNEED = C::NNEED, NEXT = C::NEXT;
  extern __shared__ __align__(16) float sm[];
  const int D = p.D, N = p.N, T = p.T, B = p.B, GD = Gr * D;
  const int tid = threadIdx.x, n = blockIdx.y, b0 = blockIdx.x * XBT;
  const size_t ND = (size_t)N * D;
  float* delta = sm;               // [8][GD]  deltas of the R-connected gates of the current step
  float* rec = delta + XBT * GD;   // [8][D]   matrix part of dh_{t-1}
  float* dbs = rec + XBT * D;      // [Gt][D]  bias gradient of this CTA's rows
  for (int i = tid; i < XBT * GD; i += XTHREADS) delta[i] = 0.f;
  for (int i = tid; i < XBT * D; i += XTHREADS) {
    rec[i] = 0.f;
    const int bl = i / D, d = i - bl * D, b = b0 + bl;
    if (b < B)  // the carried cotangents live in the ds0 output
      for (int s = 0; s < S; ++s) p.ds0[((size_t)s * B + b) * ND + (size_t)n * D + d] = 0.f;
  }
  for (int i = tid; i < Gt * D; i += XTHREADS) dbs[i] = 0.f;
  __syncthreads();
  const float* Rn = p.R + (size_t)n * D * D;  // + g * N * D * D
  for (int t = T - 1; t >= 0; --t) {
    for (int i = tid; i < XBT * D; i += XTHREADS) {
      const int bl = i / D, d = i - bl * D, b = b0 + bl;
      if (b >= B) continue;
      const size_t nd = (size_t)n * D + d;
      float car[S], dext[NEXT], cv[GCA], cur[NNEED], prv[NNEED], dR_[Gr], dW_[Gw], dB_[Gt];
#pragma unroll
      for (int s = 0; s < S; ++s) car[s] = p.ds0[((size_t)s * B + b) * ND + nd];
#pragma unroll
      for (int k = 0; k < NEXT; ++k) dext[k] = p.dstates[(size_t)k * p.ds_ss + (size_t)b * p.ds_sb + (size_t)t * p.ds_st + (size_t)n * p.ds_sn + d];
#pragma unroll
      for (int k = 0; k < GC; ++k) cv[k] = p.cache[(((size_t)b * T + t) * GCA + k) * ND + nd];
#pragma unroll
      for (int k = 0; k < NNEED; ++k) {
        const int s = C::need(k);
        cur[k] = p.states[(((size_t)s * B + b) * T + t) * ND + nd];
        prv[k] = t > 0 ? p.states[(((size_t)s * B + b) * T + (t - 1)) * ND + nd] : p.s0[((size_t)s * B + b) * ND + nd];
      }
      float r = car[0] + (p.grad_cut ? 0.f : rec[i]);
      if (p.gclip > 0.f) r = clampf(r, p.gclip);
      cell_backward<CELL>(dext[0] + r, dext, car, cv, cur, prv, dR_, dW_, dB_);
#pragma unroll
      for (int s = 0; s < S; ++s) p.ds0[((size_t)s * B + b) * ND + nd] = car[s];
#pragma unroll
      for (int g = 0; g < Gr; ++g) delta[bl * GD + g * D + d] = dR_[g];
#pragma unroll
      for (int g = 0; g < Gw; ++g) p.dWx[(((size_t)b * T + t) * Gw + g) * ND + nd] = dW_[g];
      if (CELL == CELL_GRU) p.dg0[((size_t)b * T + t) * ND + nd] = dR_[0];
#pragma unroll
      for (int g = 0; g < Gt; ++g) atomicAdd(&dbs[g * D + d], dB_[g]);
    }
    __syncthreads();
    for (int pc = tid; pc < D; pc += XTHREADS) {  // rec[b][p] = sum_{g,d} delta[b][g,d] * R[g][n][d][p]
      float acc[XBT];
#pragma unroll
      for (int b = 0; b < XBT; ++b) acc[b] = 0.f;
#pragma unroll
      for (int g = 0; g < Gr; ++g) col_dot8(Rn + (size_t)g * N * D * D, (size_t)D, pc, delta + g * D, GD, D, acc);
#pragma unroll
      for (int b = 0; b < XBT; ++b) rec[b * D + pc] = acc[b];
    }
    __syncthreads();
  }
  // cotangent of the initial h: the direct part carried in ds0[0] plus the matrix part of the last step
  for (int i = tid; i < XBT * D; i += XTHREADS) {
    const int bl = i / D, d = i - bl * D, b = b0 + bl;
    if (b < B && !p.grad_cut) p.ds0[(size_t)b * ND + (size_t)n * D + d] += rec[i];
  }
  for (int i = tid; i < Gt * D; i += XTHREADS) {
    const int g = i / D, d = i - g * D;
    atomicAdd(p.dbias + (size_t)g * ND + (size_t)n * D + d, dbs[i]);
  }
}

// ================================================================================================ cluster loops
// Shared memory of the forward loop (floats): Rs[D][Gr*U] | h[2][D][8] | part[KS][8][Gr*U] | 2 mbarriers + flag
// Rs[k][g*U + u] = R[g][n][unit0 + u][k];  h[x][k][b] = h of unit k, batch row b (CTA c's slice = rows c*U .. c*U+U-1)
// BT consecutive floats (one k, all batch rows of the tile)
template <int BT> __device__ __forceinline__ void load_row(const float* q, float (&v)[BT]) {
  if constexpr (BT == 8) {
    const float4 a = *reinterpret_cast<const float4*>(q), b = *reinterpret_cast<const float4*>(q + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else if constexpr (BT == 4) {
    const float4 a = *reinterpret_cast<const float4*>(q);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  } else {
    const float2 a = *reinterpret_cast<const float2*>(q);
    v[0] = a.x; v[1] = a.y;
  }
}

// BT = batch rows per cluster (8, 4 or 2: small batches are cut into more tiles so that more SMs take part)
template <int CELL, int IPT, int BT>
__global__ void __launch_bounds__(XTHREADS, 1) x32c_fwd_kernel(const XParams p) {
  using C = Cell<CELL>;
  constexpr int Gr = C::Gr, Gw = C::Gw, Gt = C::Gt, S = C::S, GC = C::GC, GCA = GC > 0 ? GC : 1;
  extern __shared__ __align__(16) float sm[];
  const int D = p.D, U = p.U, CS = p.CS, KS = p.KS, GU = Gr * U, T = p.T, B = p.B, N = p.N;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, b0 = blockIdx.y * BT;
  const uint32_t crank = CS > 1 ? cluster_ctarank() : 0u;
  const int unit0 = (int)crank * U;
  const size_t ND = (size_t)N * D;
  float* Rs = sm;
  float* hbuf = Rs + (size_t)D * GU;
  float* part = hbuf + 2 * BT * D;
  uint64_t* full = reinterpret_cast<uint64_t*>(part + (size_t)KS * BT * GU);
  volatile int* gave_up = reinterpret_cast<volatile int*>(full + 2);

  {  // this CTA's slice of R, from the transposed copy RT[n][k][g*D + d]
    const float* RT = p.RT + (size_t)n * D * Gr * D;
    for (int i = tid; i < D * GU; i += XTHREADS) {
      const int k = i / GU, j = i - k * GU, g = j / U, u = j - g * U;
      Rs[i] = RT[(size_t)k * Gr * D + g * D + unit0 + u];
    }
  }
  // ---- this thread's items (batch row, unit): fixed for all steps
  bool it_on[IPT], it_ok[IPT];
  int bl_[IPT], u_[IPT];
  const float* wx_p[IPT];
  float* st_p[IPT];
  float* ch_p[IPT];
  float bias[IPT][Gt], st[IPT][S], wxn[IPT][Gw];
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int q = tid + i * XTHREADS;
    it_on[i] = q < BT * U;
    bl_[i] = it_on[i] ? q / U : 0;
    u_[i] = it_on[i] ? q - bl_[i] * U : 0;
    const int bg = b0 + bl_[i], d = unit0 + u_[i];
    it_ok[i] = it_on[i] && bg < B;
    const int bgc = bg < B ? bg : B - 1;
    const size_t nd = (size_t)n * D + d;
    wx_p[i] = p.Wx + (size_t)bgc * p.wx_sb + (size_t)n * p.wx_sn + d;
    st_p[i] = p.states + ((size_t)bgc * T) * ND + nd;
    ch_p[i] = p.cache + ((size_t)bgc * T) * GCA * ND + nd;
#pragma unroll
    for (int g = 0; g < Gt; ++g) bias[i][g] = p.bias[(size_t)g * ND + nd];
#pragma unroll
    for (int s = 0; s < S; ++s) st[i][s] = it_ok[i] ? p.s0[((size_t)s * B + bg) * ND + nd] : 0.f;
#pragma unroll
    for (int g = 0; g < Gw; ++g) wxn[i][g] = it_ok[i] ? wx_p[i][(size_t)g * p.wx_sg] : 0.f;  // Wx of step 0
    wx_p[i] += p.wx_st;
  }
  // ---- h_{-1} of the whole head -> h[0] (read straight from global by every CTA)
  for (int i = tid; i < BT * D; i += XTHREADS) {
    const int bl = i / D, k = i - bl * D, b = b0 + bl;
    hbuf[k * BT + bl] = b < B ? p.s0[(size_t)b * ND + (size_t)n * D + k] : 0.f;
  }
  const uint32_t slice_bytes = (uint32_t)(U * BT * 4);
  const uint32_t expect_bytes = (uint32_t)(CS - 1) * slice_bytes;
  bool poisoned = false;
  if (CS > 1) {
    if (tid == 0) {
      *gave_up = 0;
      mbar_init(&full[0], 1);
      mbar_init(&full[1], 1);
      fence_mbar_init();
      if (T > 1) mbar_arrive_expect_tx(&full[1], expect_bytes);  // h_0, consumed at step 1
      if (T > 2) mbar_arrive_expect_tx(&full[0], expect_bytes);  // h_1, consumed at step 2
    }
    cluster_arrive();
    cluster_wait();  // every CTA of the cluster is resident and its barriers are initialised
  } else {
    __syncthreads();
  }
  const uint32_t my_slice0 = smem_u32(hbuf + (size_t)unit0 * BT);
  const uint32_t buf_bytes = (uint32_t)(BT * D * 4);
  const uint32_t full_u32 = smem_u32(&full[0]);
  // Matrix phase: a thread keeps TM gate rows x BT batch rows of sums over its share of k.  Shared memory delivers one
  // 32-bit word per lane and wavefront whatever the width of the load, so a step costs TM + BT wavefronts per TM * BT
  // FFMA of a warp: 4 x 8 sums per thread instead of 2 x 8 took 12 % off the loop of LSTM B16 N4 D256.
  constexpr int TM = BT == 8 ? 4 : 2;  // (smaller tiles: more k-splits would cost the cell phase more than the loads save)
  const int nrg = GU / TM, nwork = nrg * KS, KQ = (D + KS - 1) / KS;
  for (int t = 0; t < T; ++t) {
    const int cur = t & 1, nxt = cur ^ 1;
    float wxc[IPT][Gw];
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
#pragma unroll
      for (int g = 0; g < Gw; ++g) wxc[i][g] = wxn[i][g];
      if (it_ok[i] && t + 1 < T) {  // the next step's inputs, a whole step ahead of their use
#pragma unroll
        for (int g = 0; g < Gw; ++g) wxn[i][g] = wx_p[i][(size_t)g * p.wx_sg];
        wx_p[i] += p.wx_st;
      }
    }
    if (CS > 1 && t > 0) {
      if (!mbar_wait_bounded(&full[cur], ((t - 1) >> 1) & 1)) {
        poisoned = true;
        *gave_up = 1;
        report_timeout(p.status, t);
      }
      // re-arm for h_{t+1}; never after an expired wait: that phase is still open and has no arrival left to give
      if (tid == 0 && !poisoned && t + 2 < T) mbar_arrive_expect_tx(&full[cur], expect_bytes);
    }
    // ---------------- matrix phase: part[kc][b][row] = sum over this thread's k of R[row][k] * h_{t-1}[b][k]
    {
      const float* hcur = hbuf + (size_t)cur * BT * D;
      for (int w = tid; w < nwork; w += XTHREADS) {
        const int kc = w / nrg, rg = w - kc * nrg;
        const int k0 = kc * KQ, k1 = (k0 + KQ < D) ? k0 + KQ : D;
        float acc[TM][BT];
#pragma unroll
        for (int r = 0; r < TM; ++r)
#pragma unroll
          for (int b = 0; b < BT; ++b) acc[r][b] = 0.f;
        const float* rr = Rs + TM * rg;
#pragma unroll(TM == 4 ? 2 : 4)
        for (int k = k0; k < k1; ++k) {
          float rv[TM], hv[BT];
          load_row<TM>(rr + (size_t)k * GU, rv);
          load_row<BT>(hcur + k * BT, hv);
#pragma unroll
          for (int r = 0; r < TM; ++r)
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[r][b] = fmaf(rv[r], hv[b], acc[r][b]);
        }
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          float* dst = part + ((size_t)kc * BT + b) * GU + TM * rg;
          if constexpr (TM == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0][b], acc[1][b], acc[2][b], acc[3][b]);
          else *reinterpret_cast<float2*>(dst) = make_float2(acc[0][b], acc[1][b]);
        }
      }
    }
    __syncthreads();
    // set when a wait of this step expired in some thread of the CTA (written before the barrier above)
    const int quit = (CS > 1) ? *gave_up : 0;
    // ---------------- cell phase: this thread's items; new h into this CTA's slice of h[nxt]
    float cch[IPT][GCA];
    float* hdst = hbuf + (size_t)nxt * BT * D + (size_t)unit0 * BT;
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_on[i]) continue;
      float prv[Gr];
#pragma unroll
      for (int g = 0; g < Gr; ++g) prv[g] = 0.f;
      for (int kc = 0; kc < KS; ++kc) {
        const float* pp = part + ((size_t)kc * BT + bl_[i]) * GU + u_[i];
#pragma unroll
        for (int g = 0; g < Gr; ++g) prv[g] += pp[g * U];
      }
      cell_forward<CELL>(prv, wxc[i], bias[i], st[i], cch[i]);
      if (p.fclip > 0.f) st[i][0] = clampf(st[i][0], p.fclip);
      if (!it_ok[i]) {  // rows beyond B: keep everything zero
#pragma unroll
        for (int s = 0; s < S; ++s) st[i][s] = 0.f;
      }
      hdst[u_[i] * BT + bl_[i]] = st[i][0];
    }
    if (CS > 1) fence_proxy_async_smem();  // make the slice visible to the bulk-copy engine
    __syncthreads();
    // ---------------- push: this CTA's slice of h_t -> h[nxt] of every other CTA of the cluster
    if (CS > 1 && t + 1 < T && !(p.test_drop && crank == 0 && t == 1))  // uniform branch; one elected lane per warp copies
      push_slice_to_peers(my_slice0 + nxt * buf_bytes, slice_bytes, full_u32 + nxt * 8, crank, (uint32_t)CS, (uint32_t)warp,
                          (uint32_t)(XTHREADS >> 5));
    // ---------------- behind the exchange: results to global memory
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_ok[i]) continue;
#pragma unroll
      for (int s = 0; s < S; ++s) st_p[i][(size_t)s * B * T * ND] = st[i][s];
      st_p[i] += ND;
      if (GC > 0 && p.cache != nullptr) {
#pragma unroll
        for (int k = 0; k < GC; ++k) ch_p[i][(size_t)k * ND] = cch[i][k];
        ch_p[i] += (size_t)GCA * ND;
      }
    }
    // After an expired wait the whole CTA leaves the loop and sends nothing further, so every other CTA of the cluster
    // runs into its own bounded wait and leaves the same way.
    if (quit) break;
  }
  if (CS > 1) { cluster_arrive(); cluster_wait(); }  // no CTA leaves while a copy from or into it may be in flight
}

// Shared memory of the reverse loop (floats): Rb[Gr*U][D + 8] | delta[Gr*U][8] | send[2][CS][MSG] | recv[2][CS][MSG] |
// dbs[Gt][U] | 2 mbarriers + flag, MSG = KS*8*U.  Rb[g*U + u][p] = R[g][n][unit0 + u][p].
// Reduce-scatter: CTA c multiplies ITS deltas with its rows of R for all D columns p and sends the owner of p the
// partial sums; message for CTA x: [kc][b][u] with p = x*U + u (the CTA's own part goes straight into its recv slot).
template <int CELL, int IPT, int BT>
__global__ void __launch_bounds__(XTHREADS, 1) x32c_bwd_kernel(const XParams p) {
  using C = Cell<CELL>;
  constexpr int Gr = C::Gr, Gw = C::Gw, Gt = C::Gt, S = C::S, GC = C::GC, GCA = GC > 0 ? GC : 1, NNEED = C::NNEED, NEXT = C::NEXT;
  extern __shared__ __align__(16) float sm[];
  const int D = p.D, U = p.U, CS = p.CS, KS = p.KS, GU = Gr * U, T = p.T, B = p.B, N = p.N;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.z, b0 = blockIdx.y * BT;
  const uint32_t crank = CS > 1 ? cluster_ctarank() : 0u;
  const int unit0 = (int)crank * U;
  const size_t ND = (size_t)N * D;
  const int MSG = KS * BT * U;
  const int DP = D + 8;  // row pitch of Rb
  float* Rb = sm;
  float* delta = Rb + (size_t)GU * DP;
  float* send = delta + GU * BT;
  float* recv = send + 2 * CS * MSG;
  float* dbs = recv + 2 * CS * MSG;
  uint64_t* full = reinterpret_cast<uint64_t*>(dbs + Gt * U);
  volatile int* gave_up = reinterpret_cast<volatile int*>(full + 2);
  const bool exch = !p.grad_cut;  // with the recurrent gradient cut no dh crosses a step: no matrix phase, no exchange

  for (int i = tid; i < GU * D; i += XTHREADS) {
    const int j = i / D, pc = i - j * D, g = j / U, u = j - g * U;
    Rb[(size_t)j * DP + pc] = p.R[(((size_t)g * N + n) * D + unit0 + u) * D + pc];
  }
  for (int i = tid; i < Gt * U; i += XTHREADS) dbs[i] = 0.f;

  bool it_on[IPT], it_ok[IPT];
  int bl_[IPT], u_[IPT];
  const float* st_p[IPT];   // states[0][b][t][n][d] of the step whose values are loaded NEXT
  const float* ch_p[IPT];
  const float* ex_p[IPT];
  float* dw_p[IPT];
  float* dg_p[IPT];
  float car[IPT][S], cur[IPT][NNEED], prv[IPT][NNEED], cv[IPT][GCA], ext[IPT][NEXT], dbacc[IPT][Gt];
  const size_t sstride = (size_t)B * T * ND;
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int q = tid + i * XTHREADS;
    it_on[i] = q < BT * U;
    bl_[i] = it_on[i] ? q / U : 0;
    u_[i] = it_on[i] ? q - bl_[i] * U : 0;
    const int bg = b0 + bl_[i], d = unit0 + u_[i];
    it_ok[i] = it_on[i] && bg < B;
    const int bgc = bg < B ? bg : B - 1;
    const size_t nd = (size_t)n * D + d;
    // everything of time T-1
    st_p[i] = p.states + ((size_t)bgc * T + (T - 1)) * ND + nd;
    ch_p[i] = p.cache + (((size_t)bgc * T + (T - 1)) * GCA) * ND + nd;
    ex_p[i] = p.dstates + (size_t)bgc * p.ds_sb + (size_t)(T - 1) * p.ds_st + (size_t)n * p.ds_sn + d;
    dw_p[i] = p.dWx + (((size_t)bgc * T + (T - 1)) * Gw) * ND + nd;
    dg_p[i] = p.dg0 + ((size_t)bgc * T + (T - 1)) * ND + nd;
#pragma unroll
    for (int s = 0; s < S; ++s) car[i][s] = 0.f;
#pragma unroll
    for (int g = 0; g < Gt; ++g) dbacc[i][g] = 0.f;
#pragma unroll
    for (int k = 0; k < NNEED; ++k) {
      const size_t so = (size_t)C::need(k) * sstride;
      cur[i][k] = it_ok[i] ? st_p[i][so] : 1.f;
      prv[i][k] = !it_ok[i] ? 1.f : (T > 1 ? st_p[i][so - ND] : p.s0[((size_t)C::need(k) * B + bgc) * ND + nd]);
    }
#pragma unroll
    for (int k = 0; k < GCA; ++k) cv[i][k] = (GC > 0 && it_ok[i] && k < GC) ? ch_p[i][(size_t)k * ND] : 0.f;
#pragma unroll
    for (int k = 0; k < NEXT; ++k) ext[i][k] = it_ok[i] ? ex_p[i][(size_t)k * p.ds_ss] : 0.f;
    st_p[i] -= 2 * ND;  // the next load of a previous state is the one of time T-3 (prv of step T-2)
    ch_p[i] -= (size_t)GCA * ND;
    ex_p[i] -= p.ds_st;
  }
  const uint32_t msg_bytes = (uint32_t)(MSG * 4);
  const uint32_t expect_bytes = (uint32_t)(CS - 1) * msg_bytes;
  const bool xc = exch && CS > 1;
  bool poisoned = false;
  if (CS > 1) {
    if (tid == 0) {
      *gave_up = 0;
      mbar_init(&full[0], 1);
      mbar_init(&full[1], 1);
      fence_mbar_init();
      if (exch) {
        mbar_arrive_expect_tx(&full[0], expect_bytes);             // partial sums of step 0
        if (T > 1) mbar_arrive_expect_tx(&full[1], expect_bytes);  // ... of step 1
      }
    }
    cluster_arrive();
    cluster_wait();
  } else {
    __syncthreads();
  }
  const uint32_t full_u32 = smem_u32(&full[0]);
  const int ncg8 = (D + 31) >> 5, ntasks = ncg8 * KS, KQ = ((GU + KS - 1) / KS + 3) & ~3;  // rows per k-split, a multiple of 4

  // sum of the partial sums that arrived for item i in buffer x
  auto gather = [&](int i, int x) {
    float r = 0.f;
    for (int c = 0; c < CS; ++c) {
      const float* q = recv + ((size_t)x * CS + c) * MSG + bl_[i] * U + u_[i];
      for (int kc = 0; kc < KS; ++kc) r += q[(size_t)kc * BT * U];
    }
    return r;
  };
  bool quit_all = false;
  for (int j = 0; j < T; ++j) {  // j-th step of the reverse loop, time t = T-1-j
    const int t = T - 1 - j, buf = j & 1, pb = buf ^ 1;
    // ---- the next step's inputs (time t-1), a whole step ahead of their use
    float prv_n[IPT][NNEED], cv_n[IPT][GCA], ext_n[IPT][NEXT];
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
#pragma unroll
      for (int k = 0; k < NNEED; ++k) prv_n[i][k] = 1.f;
#pragma unroll
      for (int k = 0; k < GCA; ++k) cv_n[i][k] = 0.f;
#pragma unroll
      for (int k = 0; k < NEXT; ++k) ext_n[i][k] = 0.f;
      if (it_ok[i] && t > 0) {
        const int bg = b0 + bl_[i];
        const size_t nd = (size_t)n * D + unit0 + u_[i];
#pragma unroll
        for (int k = 0; k < NNEED; ++k)
          prv_n[i][k] = t > 1 ? st_p[i][(size_t)C::need(k) * sstride] : p.s0[((size_t)C::need(k) * B + bg) * ND + nd];
        if (GC > 0) {
#pragma unroll
          for (int k = 0; k < GC; ++k) cv_n[i][k] = ch_p[i][(size_t)k * ND];
        }
#pragma unroll
        for (int k = 0; k < NEXT; ++k) ext_n[i][k] = ex_p[i][(size_t)k * p.ds_ss];
        st_p[i] -= ND;
        ch_p[i] -= (size_t)GCA * ND;
        ex_p[i] -= p.ds_st;
      }
    }
    if (xc && j > 0) {  // the partial sums of step j-1
      if (!mbar_wait_bounded(&full[pb], ((j - 1) >> 1) & 1)) {
        poisoned = true;
        *gave_up = 1;
        report_timeout(p.status, t);
      }
      if (tid == 0 && !poisoned && j + 1 < T) mbar_arrive_expect_tx(&full[pb], expect_bytes);  // re-arm for step j+1
    }
    // ---------------- cell phase
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_on[i]) continue;
      float r = car[i][0];
      if (exch && j > 0) r += gather(i, pb);
      if (p.gclip > 0.f) r = clampf(r, p.gclip);
      float dR_[Gr], dW_[Gw], dB_[Gt];
      cell_backward<CELL>(ext[i][0] + r, ext[i], car[i], cv[i], cur[i], prv[i], dR_, dW_, dB_);
      if (!it_ok[i]) {
#pragma unroll
        for (int s = 0; s < S; ++s) car[i][s] = 0.f;
#pragma unroll
        for (int g = 0; g < Gr; ++g) dR_[g] = 0.f;
      } else {
#pragma unroll
        for (int g = 0; g < Gw; ++g) dw_p[i][(size_t)g * ND] = dW_[g];
        dw_p[i] -= (size_t)Gw * ND;
        if (CELL == CELL_GRU) { *dg_p[i] = dR_[0]; dg_p[i] -= ND; }
#pragma unroll
        for (int g = 0; g < Gt; ++g) dbacc[i][g] += dB_[g];
      }
#pragma unroll
      for (int g = 0; g < Gr; ++g) delta[(g * U + u_[i]) * BT + bl_[i]] = dR_[g];
#pragma unroll
      for (int k = 0; k < NNEED; ++k) { cur[i][k] = prv[i][k]; prv[i][k] = prv_n[i][k]; }
#pragma unroll
      for (int k = 0; k < GCA; ++k) cv[i][k] = cv_n[i][k];
#pragma unroll
      for (int k = 0; k < NEXT; ++k) ext[i][k] = ext_n[i][k];
    }
    __syncthreads();
    const int quit = (CS > 1) ? *gave_up : 0;
    if (exch) {
      // ---------------- matrix phase: partial dh_{t-1}[b][p] = sum over this thread's (g, u) of delta[b][g,u] * R[g][u][p]
      // A warp task: 32 columns (lane >> 2 picks 4 of them) x one of the KS row ranges; inside the range lane & 3 takes
      // every fourth row, and the four sums meet again through shuffles.  4 x BT sums per thread: 4 + BT words from shared
      // memory per 4 * BT FFMA (see the forward loop), and a message stays one [BT][U] block per k-split.  Rows of Rb are
      // D + 8 words apart, so the four rows a quarter-warp reads together fall into different banks.
      for (int task = warp; task < ntasks; task += XTHREADS >> 5) {
        const int kx = task / ncg8, pc = (task - kx * ncg8) * 32 + (lane >> 2) * 4;  // columns pc .. pc+3
        const int j0 = kx * KQ + (lane & 3), j1 = ((kx + 1) * KQ < GU) ? (kx + 1) * KQ : GU;
        const bool live = pc < D;
        float acc[4][BT];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int b = 0; b < BT; ++b) acc[c][b] = 0.f;
        if (live) {
          const float* rr = Rb + pc;
#pragma unroll 2
          for (int jj = j0; jj < j1; jj += 4) {
            const float4 r = *reinterpret_cast<const float4*>(rr + (size_t)jj * DP);
            float dv[BT];
            load_row<BT>(delta + jj * BT, dv);
#pragma unroll
            for (int b = 0; b < BT; ++b) {
              acc[0][b] = fmaf(r.x, dv[b], acc[0][b]);
              acc[1][b] = fmaf(r.y, dv[b], acc[1][b]);
              acc[2][b] = fmaf(r.z, dv[b], acc[2][b]);
              acc[3][b] = fmaf(r.w, dv[b], acc[3][b]);
            }
          }
        }
        // reduce-scatter over the four lanes of a column group: lane bit 1 keeps columns {0,1} or {2,3}, bit 0 one of the two
        const bool hi1 = (lane & 2) != 0, hi0 = (lane & 1) != 0;
        float two[2][BT], one[BT];
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          const float s0 = hi1 ? acc[0][b] : acc[2][b], s1 = hi1 ? acc[1][b] : acc[3][b];
          const float g0 = __shfl_xor_sync(0xffffffffu, s0, 2), g1 = __shfl_xor_sync(0xffffffffu, s1, 2);
          two[0][b] = (hi1 ? acc[2][b] : acc[0][b]) + g0;
          two[1][b] = (hi1 ? acc[3][b] : acc[1][b]) + g1;
        }
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          const float s = hi0 ? two[0][b] : two[1][b];
          const float g = __shfl_xor_sync(0xffffffffu, s, 1);
          one[b] = (hi0 ? two[1][b] : two[0][b]) + g;
        }
        if (live) {
          const int pcol = pc + (hi1 ? 2 : 0) + (hi0 ? 1 : 0);
          const int c = pcol / U, u = pcol - c * U;
          // the owner's slot: recv[buf][crank] over there; the message leaves from send[buf][c], the own part stays here
          float* dst = ((uint32_t)c == crank ? recv + ((size_t)buf * CS + crank) * MSG : send + ((size_t)buf * CS + c) * MSG) +
                       (size_t)kx * BT * U + u;
#pragma unroll
          for (int b = 0; b < BT; ++b) dst[b * U] = one[b];
        }
      }
      if (CS > 1) fence_proxy_async_smem();
      __syncthreads();
      if (CS > 1 && !(p.test_drop && crank == 0 && j == 1)) {  // uniform branch; warp w serves the peers w, w + 8, ...
        __syncwarp();
        for (uint32_t c = (uint32_t)warp; c < (uint32_t)CS; c += XTHREADS >> 5) {
          if (c == crank) continue;
          const uint32_t src = smem_u32(send + ((size_t)buf * CS + c) * MSG);
          const uint32_t dst = map_to_cta(smem_u32(recv + ((size_t)buf * CS + crank) * MSG), c);
          const uint32_t bar = map_to_cta(full_u32 + buf * 8, c);
          if (elect_one_sync()) bulk_copy_to_cta(dst, src, msg_bytes, bar);
        }
      }
    }
    if (quit) { quit_all = true; break; }
  }
  // ---- cotangents of the initial states: the carried ones; h also gets the matrix part of the last step
  if (xc && !quit_all) {
    if (!mbar_wait_bounded(&full[(T - 1) & 1], ((T - 1) >> 1) & 1)) {
      report_timeout(p.status, -1);
      quit_all = true;
    }
  }
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    if (!it_ok[i]) continue;
    const int bg = b0 + bl_[i];
    const size_t nd = (size_t)n * D + unit0 + u_[i];
    float r = car[i][0];
    if (exch && !quit_all) r += gather(i, (T - 1) & 1);
    p.ds0[(size_t)bg * ND + nd] = r;
#pragma unroll
    for (int s = 1; s < S; ++s) p.ds0[((size_t)s * B + bg) * ND + nd] = car[i][s];
#pragma unroll
    for (int g = 0; g < Gt; ++g) atomicAdd(&dbs[g * U + u_[i]], dbacc[i][g]);
  }
  __syncthreads();
  for (int i = tid; i < Gt * U; i += XTHREADS) {
    const int g = i / U, u = i - g * U;
    atomicAdd(p.dbias + (size_t)g * ND + (size_t)n * D + unit0 + u, dbs[i]);
  }
  if (CS > 1) { cluster_arrive(); cluster_wait(); }
}

// dR[g][n][d][p] += sum over this CTA's rows k = (b, t) of delta_g[k][d] * h_{t-1}[k][p]: a 128 x 64 tile of ((g, d), p),
// 8 x 4 sums per thread, 16 rows of k per stage (the next stage's global loads are in flight while this one is multiplied),
// split-K over the grid's z, fp32 atomics at the end.
struct XDrParams {
  const float* dWx; const float* dg0; const float* states; const float* s0; float* dR;
  int cell, B, T, N, D, Gr, Gw;
  long long K;
  int rows_per_split;
};
constexpr int DR_M = 128, DR_P = 64, DR_K = 16;
__global__ void __launch_bounds__(XTHREADS) x32_dr_kernel(const XDrParams p) {
  __shared__ __align__(16) float As[2][DR_K][DR_M];
  __shared__ __align__(16) float Hs[2][DR_K][DR_P];
  const int D = p.D, N = p.N, T = p.T, GD = p.Gr * D;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * DR_M, p0 = blockIdx.y * DR_P;
  const int n = blockIdx.z % N, split = blockIdx.z / N;
  const size_t ND = (size_t)N * D;
  const long long k0 = (long long)split * p.rows_per_split;
  long long k1 = k0 + p.rows_per_split;
  if (k1 > p.K) k1 = p.K;
  // global -> register staging: thread loads A chunks (kk = tid / 32 + {0, 8}, 4 columns at (tid % 32) * 4) and one H chunk
  const int a_kk = tid >> 5, a_c = (tid & 31) * 4;
  const int h_kk = tid >> 4, h_c = (tid & 15) * 4;
  const float* a_src[2];  // per A chunk: address of (k = 0) or null when the column is outside the matrix
  {
    const int m = m0 + a_c;
    const float* base = nullptr;
    if (m < GD) {
      const int g = m / D, d = m - g * D;
      if (p.cell == CELL_GRU && g == 0) base = p.dg0 + (size_t)n * D + d;
      else base = p.dWx + (size_t)(p.cell == CELL_GRU ? g - 1 : g) * ND + (size_t)n * D + d;
    }
    a_src[0] = a_src[1] = base;
  }
  const bool a_dg0 = p.cell == CELL_GRU && (m0 + a_c) < D;
  const size_t a_row = a_dg0 ? ND : (size_t)p.Gw * ND;  // floats between rows k and k+1
  const bool h_on = p0 + h_c < D;
  float4 ra[2], rh;
  auto fetch = [&](long long kc) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const long long k = kc + a_kk + 8 * i;
      ra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < k1 && a_src[i] != nullptr) ra[i] = *reinterpret_cast<const float4*>(a_src[i] + (size_t)k * a_row);
    }
    const long long k = kc + h_kk;
    rh = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < k1 && h_on) {
      const long long b = k / T;
      const int tt = (int)(k - b * T);
      const float* src = tt > 0 ? p.states + (size_t)(k - 1) * ND : p.s0 + (size_t)b * ND;
      rh = *reinterpret_cast<const float4*>(src + (size_t)n * D + p0 + h_c);
    }
  };
  auto stash = [&](int s) {
    *reinterpret_cast<float4*>(&As[s][a_kk][a_c]) = ra[0];
    *reinterpret_cast<float4*>(&As[s][a_kk + 8][a_c]) = ra[1];
    *reinterpret_cast<float4*>(&Hs[s][h_kk][h_c]) = rh;
  };
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  fetch(k0);
  stash(0);
  __syncthreads();
  int s = 0;
  for (long long kc = k0; kc < k1; kc += DR_K) {
    const bool more = kc + DR_K < k1;
    if (more) fetch(kc + DR_K);
#pragma unroll
    for (int kk = 0; kk < DR_K; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[s][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[s][kk][64 + ty * 4]);
      const float4 h4 = *reinterpret_cast<const float4*>(&Hs[s][kk][tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float hh[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], hh[j], acc[i][j]);
    }
    if (more) stash(s ^ 1);
    __syncthreads();
    s ^= 1;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= GD) continue;
    const int g = m / D, d = m - g * D;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pc = p0 + tx * 4 + j;
      if (pc < D) atomicAdd(p.dR + (((size_t)g * N + n) * D + d) * D + pc, acc[i][j]);
    }
  }
}

struct Dims { int Gr, Gw, Gt, S, GC; };
bool dims_of(int cell, float fclip, Dims* d) {
  switch (cell) {
    case CELL_LSTM: *d = {4, 4, 4, 2, 4}; return true;
    case CELL_GRU: *d = {3, 3, 4, 1, 4}; return true;
    case CELL_ELMAN: *d = {1, 1, 1, 1, fclip > 0.f ? 1 : 0}; return true;
    case CELL_SLSTM: *d = {4, 4, 4, 4, 5}; return true;
  }
  return false;
}
size_t up256(size_t x) { return (x + 255) / 256 * 256; }
struct Ws { size_t rt, grads, dg0, total; };
Ws ws_layout(const frnn_problem& pr, const Dims& d) {
  Ws w;
  size_t off = kStatus;
  w.rt = off; off = up256(off + (size_t)d.Gr * pr.N * pr.D * pr.D * 4);
  w.grads = off; off = up256(off + ((size_t)d.Gr * pr.N * pr.D * pr.D + (size_t)d.Gt * pr.N * pr.D) * 4);
  w.dg0 = off;
  if (pr.cell == CELL_GRU) off = up256(off + (size_t)pr.B * pr.T * pr.N * pr.D * 4);
  w.total = off;
  return w;
}
size_t fwd_smem(const frnn_problem& pr, const Dims& d, bool r_in) {
  return ((size_t)XBT * pr.D + (size_t)XBT * d.Gr * pr.D + (r_in ? (size_t)pr.D * d.Gr * pr.D : 0)) * 4;
}
size_t bwd_smem(const frnn_problem& pr, const Dims& d) {
  return ((size_t)XBT * d.Gr * pr.D + (size_t)XBT * pr.D + (size_t)d.Gt * pr.D) * 4;
}
// Geometry of the loops for a cluster size: U units per CTA, k-splits of the two matrix phases, items per thread.
// `cluster` false = the streamed loops (one CTA per head, R from L2).
struct Tile { int cs, u, bt, ksf, ksb, ipt; bool cluster; size_t smem_f, smem_b; };
int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
// Clusters of one CTA per SM that a B200 (148 SMs in GPCs of unequal size) keeps resident at once, by cluster size, as
// cudaOccupancyMaxActiveClusters reports it for these kernels' footprint (sizes 5 and 7: not measured, rounded down).
constexpr int kResidentClusters[9] = {0, 148, 74, 45, 33, 26, 22, 17, 15};
// bt == 0: the smallest batch tile (8, 4, 2 rows) whose clusters are still all resident at once -- within one wave the
// step time falls with the rows per CTA, beyond it the tiles queue up (LSTM B16 N4 D256: 16 clusters of 8 ran 25 % slower
// than 8 clusters of twice the rows)
bool cluster_tile(const frnn_problem& pr, const Dims& d, int cs, int bt, Tile* t) {
  if (cs < 1 || cs > 8 || pr.D % cs) return false;
  if (bt != 0 && bt != 8 && bt != 4 && bt != 2) return false;
  const int u = pr.D / cs;
  if (u % 4 || u > 64) return false;
  const size_t gu = (size_t)d.Gr * u, D = (size_t)pr.D;
  if (bt == 0) {
    bt = 8;
    while (bt > 2 && (long long)((pr.B + bt / 2 - 1) / (bt / 2)) * pr.N <= kResidentClusters[cs]) bt /= 2;
  }
  t->cs = cs; t->u = u; t->bt = bt; t->cluster = true;
  const int tm = bt == 8 ? 4 : 2;  // gate rows per thread in the forward matrix phase
  t->ksf = clampi((int)(XTHREADS * tm / gu), 1, clampi((int)(32768 / (bt * gu * 4)), 1, 16));  // partial sums within 32 KB
  t->ksb = clampi((XTHREADS / 32) / ((pr.D + 31) / 32), 1, 8);  // warp tasks of 32 columns: as many row ranges as fill the warps
  t->ipt = bt * u > XTHREADS ? 2 : 1;
  t->smem_f = (D * gu + 2 * bt * D + (size_t)t->ksf * bt * gu) * 4 + 64;
  t->smem_b = (gu * (D + 8) + gu * bt + (size_t)4 * t->ksb * bt * D + (size_t)d.Gt * u) * 4 + 64;
  return t->smem_f <= kSmemMax && t->smem_b <= kSmemMax;
}
// cs == 0: the preferred tile -- the whole head in one CTA up to head dim 64, else the smallest cluster with at most 32
// units per CTA, else the smallest cluster that fits, else the streamed loops.  cs > 0: that cluster size or nothing
// (cs == 1 falls back to the streamed loops when the head does not fit one CTA).
bool pick_tile(const frnn_problem& pr, const Dims& d, int cs, int bt, Tile* t) {
  if (cs > 0) {
    if (cluster_tile(pr, d, cs, bt, t)) return true;
    if (cs != 1) return false;
  } else {
    if (pr.D <= 64 && cluster_tile(pr, d, 1, bt, t)) return true;
    for (int c = 1; c <= 8; ++c)
      if (cluster_tile(pr, d, c, bt, t) && t->u <= 32) return true;
    for (int c = 1; c <= 8; ++c)
      if (cluster_tile(pr, d, c, bt, t)) return true;
  }
  if (bt != 0 && bt != XBT) return false;  // the streamed loops work on 8 rows
  *t = Tile{1, pr.D, XBT, 0, 0, 0, false, fwd_smem(pr, d, false), bwd_smem(pr, d)};
  return t->smem_f <= kSmemMax && t->smem_b <= kSmemMax;
}
int validate(const frnn_problem* pr, Dims* d) {
  if (!pr) return FRNN_ERR_NULL;
  if (!dims_of(pr->cell, pr->forward_clip, d)) return FRNN_ERR_CELL;
  if (pr->dtype_io != FRNN_DTYPE_F32 || pr->dtype_state != FRNN_DTYPE_F32) return FRNN_ERR_DTYPE;
  if (pr->B < 1 || pr->T < 1 || pr->N < 1 || pr->N > 65535 || pr->D < 4 || pr->D > 1024 || pr->D % 4) return FRNN_ERR_SHAPE;
  if ((pr->B + XBT - 1) / XBT > 65535) return FRNN_ERR_SHAPE;
  Tile t;
  if (!pick_tile(*pr, *d, 0, 0, &t)) return FRNN_ERR_SHAPE;
  return FRNN_OK;
}
int check(const frnn_plan* pl, Dims* d, Tile* t) {
  if (!pl) return FRNN_ERR_NULL;
  if (pl->abi_version != FRNN_ABI_VERSION) return FRNN_ERR_PLAN;
  const int rc = validate(&pl->prob, d);
  if (rc) return rc;
  if (!pick_tile(pl->prob, *d, pl->cluster_size, pl->batch_tile, t) || pl->threads != XTHREADS ||
      pl->units_per_cta != t->u || pl->workspace_bytes != ws_layout(pl->prob, *d).total || pl->probe_noop_cell)
    return FRNN_ERR_PLAN;
  return FRNN_OK;
}
template <typename K>
cudaError_t launch_cluster(K kern, const frnn_problem& pr, const Tile& t, size_t smem, const XParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax);  // fixed maximum
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)t.cs, (unsigned)((pr.B + t.bt - 1) / t.bt), (unsigned)pr.N);
  cfg.blockDim = dim3(XTHREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)t.cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = t.cs > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool strides_ok(const int64_t (&in)[4], const long long (&dense)[4], long long (&out)[4]) {
  const bool zero = !in[0] && !in[1] && !in[2] && !in[3];
  for (int i = 0; i < 4; ++i) {
    if (!zero && (in[i] < 0 || in[i] % 8)) return false;
    out[i] = zero ? dense[i] : in[i];
  }
  return true;
}
template <typename K> cudaError_t set_smem(K kern) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax);  // fixed maximum
}

}  // namespace
}  // namespace FRNN_NS

using namespace FRNN_NS;

extern "C" {

__attribute__((visibility("hidden"))) int frnn_query_f32(const frnn_problem* pr, int cs, int bt, int stages, frnn_plan* out) {
  Dims d;
  const int rc = validate(pr, &d);
  if (rc) return rc;
  if (!out) return FRNN_ERR_NULL;
  if (stages) return FRNN_ERR_PLAN;  // no input ring
  Tile tl;
  if (!pick_tile(*pr, d, cs, bt, &tl)) return FRNN_ERR_PLAN;
  frnn_plan pl = {};
  pl.abi_version = FRNN_ABI_VERSION;
  pl.prob = *pr;
  pl.cluster_size = tl.cs;
  pl.units_per_cta = tl.u;
  pl.batch_tile = tl.bt;
  pl.threads = XTHREADS;
  pl.wx_stages = 0;
  pl.cache_slots = d.GC;
  pl.cache_bytes = (uint64_t)pr->B * pr->T * d.GC * pr->N * pr->D * 4;
  const Ws w = ws_layout(*pr, d);
  pl.workspace_bytes = w.total;
  pl.grads_offset = w.grads;
  pl.grads_count = (uint64_t)d.Gr * pr->N * pr->D * pr->D + (uint64_t)d.Gt * pr->N * pr->D;
  *out = pl;
  return FRNN_OK;
}

__attribute__((visibility("hidden"))) int frnn_forward_f32(const frnn_plan* plan, const frnn_fwd_args* a, void* stream_) {
  Dims d;
  Tile tl;
  int rc = check(plan, &d, &tl);
  if (rc) return rc;
  const frnn_problem& pr = plan->prob;
  if (!a || !a->Wx || !a->R || !a->b || !a->s0 || !a->states || !a->workspace) return FRNN_ERR_NULL;
  if (pr.training && d.GC > 0 && !a->cache) return FRNN_ERR_NULL;
  if (!aligned16(a->Wx) || !aligned16(a->R) || !aligned16(a->b) || !aligned16(a->s0) || !aligned16(a->states) ||
      !aligned16(a->workspace) || (a->cache && !aligned16(a->cache)) || (a->last && !aligned16(a->last)))
    return FRNN_ERR_ALIGN;
  const long long nd = (long long)pr.N * pr.D;
  const long long wx_dense[4] = {(long long)pr.T * d.Gw * nd, d.Gw * nd, nd, pr.D};
  long long wxs[4];
  if (!strides_ok(a->wx_stride, wx_dense, wxs)) return FRNN_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  const Ws w = ws_layout(pr, d);
  cudaError_t e = cudaSuccess;
  if (!plan->keep_packed_r) {
    e = cudaMemsetAsync(ws, 0, kStatus, stream);
    if (e != cudaSuccess) return (int)e;
    const size_t total = (size_t)d.Gr * pr.N * pr.D * pr.D;
    transpose_recurrent_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(static_cast<const float*>(a->R),
                                                                                   reinterpret_cast<float*>(ws + w.rt), d.Gr, pr.N, pr.D);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  XParams p = {};
  p.Wx = static_cast<const float*>(a->Wx); p.R = static_cast<const float*>(a->R); p.RT = reinterpret_cast<const float*>(ws + w.rt);
  p.bias = static_cast<const float*>(a->b); p.s0 = static_cast<const float*>(a->s0);
  p.states = static_cast<float*>(a->states); p.cache = pr.training ? static_cast<float*>(a->cache) : nullptr;
  p.B = pr.B; p.T = pr.T; p.N = pr.N; p.D = pr.D;
  p.status = reinterpret_cast<unsigned*>(ws);
  p.fclip = pr.forward_clip; p.gclip = pr.grad_clip; p.grad_cut = pr.grad_cut;
  p.wx_sb = wxs[0]; p.wx_st = wxs[1]; p.wx_sg = wxs[2]; p.wx_sn = wxs[3];
  if (tl.cluster) {
    p.U = tl.u; p.CS = tl.cs; p.KS = tl.ksf; p.test_drop = plan->test_drop_exchange;
    auto launch = [&](auto cell) {
      constexpr int CL = decltype(cell)::value;
      if (tl.ipt == 2) return launch_cluster(x32c_fwd_kernel<CL, 2, 8>, pr, tl, tl.smem_f, p, stream);
      if (tl.bt == 8) return launch_cluster(x32c_fwd_kernel<CL, 1, 8>, pr, tl, tl.smem_f, p, stream);
      if (tl.bt == 4) return launch_cluster(x32c_fwd_kernel<CL, 1, 4>, pr, tl, tl.smem_f, p, stream);
      return launch_cluster(x32c_fwd_kernel<CL, 1, 2>, pr, tl, tl.smem_f, p, stream);
    };
    using std::integral_constant;
    switch (pr.cell) {
      case CELL_LSTM: e = launch(integral_constant<int, CELL_LSTM>{}); break;
      case CELL_GRU: e = launch(integral_constant<int, CELL_GRU>{}); break;
      case CELL_SLSTM: e = launch(integral_constant<int, CELL_SLSTM>{}); break;
      default:
        e = pr.forward_clip > 0.f ? launch(integral_constant<int, CELL_ELMAN_CLIP>{}) : launch(integral_constant<int, CELL_ELMAN>{});
        break;
    }
  } else {
    p.r_in_smem = fwd_smem(pr, d, true) <= kSmemMax;
    const dim3 grid((unsigned)((pr.B + XBT - 1) / XBT), (unsigned)pr.N);
    const size_t smem = fwd_smem(pr, d, p.r_in_smem != 0);
    auto launch = [&](auto kern) -> cudaError_t {
      cudaError_t s = set_smem(kern);
      if (s != cudaSuccess) return s;
      kern<<<grid, XTHREADS, smem, stream>>>(p);
      return cudaGetLastError();
    };
    switch (pr.cell) {
      case CELL_LSTM: e = launch(x32_fwd_kernel<CELL_LSTM>); break;
      case CELL_GRU: e = launch(x32_fwd_kernel<CELL_GRU>); break;
      case CELL_SLSTM: e = launch(x32_fwd_kernel<CELL_SLSTM>); break;
      default: e = pr.forward_clip > 0.f ? launch(x32_fwd_kernel<CELL_ELMAN_CLIP>) : launch(x32_fwd_kernel<CELL_ELMAN>); break;
    }
  }
  if (e != cudaSuccess) return (int)e;
  if (a->last) {  // states[:, :, T-1] -> last (may be the s0 buffer itself)
    const size_t row = (size_t)pr.N * pr.D * 4;
    e = cudaMemcpy2DAsync(a->last, row, static_cast<const unsigned char*>(a->states) + (size_t)(pr.T - 1) * row, (size_t)pr.T * row, row,
                          (size_t)d.S * pr.B, cudaMemcpyDeviceToDevice, stream);
  }
  return (int)e;
}

__attribute__((visibility("hidden"))) int frnn_backward_parts_f32(const frnn_plan* plan, const frnn_bwd_args* a, void* stream_, int parts) {
  Dims d;
  Tile tl;
  int rc = check(plan, &d, &tl);
  if (rc) return rc;
  const frnn_problem& pr = plan->prob;
  if (!pr.training) return FRNN_ERR_TRAINING;
  if (!a || !a->R || !a->s0 || !a->states || !a->dstates || !a->dWx || !a->ds0 || !a->workspace) return FRNN_ERR_NULL;
  if (d.GC > 0 && !a->cache) return FRNN_ERR_NULL;
  if (!aligned16(a->R) || !aligned16(a->s0) || !aligned16(a->states) || !aligned16(a->dstates) || !aligned16(a->dWx) ||
      !aligned16(a->ds0) || !aligned16(a->workspace) || (a->cache && !aligned16(a->cache)))
    return FRNN_ERR_ALIGN;
  const long long nd = (long long)pr.N * pr.D;
  const long long ds_dense[4] = {(long long)pr.B * pr.T * nd, (long long)pr.T * nd, nd, pr.D};
  long long dss[4];
  if (!strides_ok(a->dstates_stride, ds_dense, dss)) return FRNN_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  const Ws w = ws_layout(pr, d);
  float* grads = reinterpret_cast<float*>(ws + w.grads);
  const size_t nR = (size_t)d.Gr * pr.N * pr.D * pr.D, nb = (size_t)d.Gt * pr.N * pr.D;
  cudaError_t e = cudaSuccess;
  if (parts & FRNN_PART_LOOP) {
    e = cudaMemsetAsync(ws, 0, kStatus, stream);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemsetAsync(grads, 0, (nR + nb) * sizeof(float), stream);
    if (e != cudaSuccess) return (int)e;
    XParams p = {};
    p.R = static_cast<const float*>(a->R); p.s0 = static_cast<const float*>(a->s0);
    p.states = static_cast<float*>(const_cast<void*>(a->states)); p.cache = static_cast<float*>(const_cast<void*>(a->cache));
    p.dstates = static_cast<const float*>(a->dstates); p.dWx = static_cast<float*>(a->dWx);
    p.dg0 = reinterpret_cast<float*>(ws + w.dg0); p.ds0 = static_cast<float*>(a->ds0); p.dbias = grads + nR;
    p.B = pr.B; p.T = pr.T; p.N = pr.N; p.D = pr.D;
    p.fclip = pr.forward_clip; p.gclip = pr.grad_clip; p.grad_cut = pr.grad_cut;
    p.ds_ss = dss[0]; p.ds_sb = dss[1]; p.ds_st = dss[2]; p.ds_sn = dss[3];
    p.status = reinterpret_cast<unsigned*>(ws);
    if (tl.cluster) {
      p.U = tl.u; p.CS = tl.cs; p.KS = tl.ksb; p.test_drop = plan->test_drop_exchange;
      auto launch = [&](auto cell) {
      constexpr int CL = decltype(cell)::value;
      if (tl.ipt == 2) return launch_cluster(x32c_bwd_kernel<CL, 2, 8>, pr, tl, tl.smem_b, p, stream);
      if (tl.bt == 8) return launch_cluster(x32c_bwd_kernel<CL, 1, 8>, pr, tl, tl.smem_b, p, stream);
      if (tl.bt == 4) return launch_cluster(x32c_bwd_kernel<CL, 1, 4>, pr, tl, tl.smem_b, p, stream);
      return launch_cluster(x32c_bwd_kernel<CL, 1, 2>, pr, tl, tl.smem_b, p, stream);
    };
    using std::integral_constant;
    switch (pr.cell) {
      case CELL_LSTM: e = launch(integral_constant<int, CELL_LSTM>{}); break;
      case CELL_GRU: e = launch(integral_constant<int, CELL_GRU>{}); break;
      case CELL_SLSTM: e = launch(integral_constant<int, CELL_SLSTM>{}); break;
      default:
        e = pr.forward_clip > 0.f ? launch(integral_constant<int, CELL_ELMAN_CLIP>{}) : launch(integral_constant<int, CELL_ELMAN>{});
        break;
    }
    } else {
      const dim3 grid((unsigned)((pr.B + XBT - 1) / XBT), (unsigned)pr.N);
      const size_t smem = bwd_smem(pr, d);
      auto launch = [&](auto kern) -> cudaError_t {
        cudaError_t s = set_smem(kern);
        if (s != cudaSuccess) return s;
        kern<<<grid, XTHREADS, smem, stream>>>(p);
        return cudaGetLastError();
      };
      switch (pr.cell) {
        case CELL_LSTM: e = launch(x32_bwd_kernel<CELL_LSTM>); break;
        case CELL_GRU: e = launch(x32_bwd_kernel<CELL_GRU>); break;
        case CELL_SLSTM: e = launch(x32_bwd_kernel<CELL_SLSTM>); break;
        default: e = pr.forward_clip > 0.f ? launch(x32_bwd_kernel<CELL_ELMAN_CLIP>) : launch(x32_bwd_kernel<CELL_ELMAN>); break;
      }
    }
    if (e != cudaSuccess) return (int)e;
  }
  if (parts & FRNN_PART_DR) {
    XDrParams q = {};
    q.dWx = static_cast<const float*>(a->dWx); q.dg0 = reinterpret_cast<const float*>(ws + w.dg0);
    q.states = static_cast<const float*>(a->states); q.s0 = static_cast<const float*>(a->s0); q.dR = grads;
    q.cell = pr.cell; q.B = pr.B; q.T = pr.T; q.N = pr.N; q.D = pr.D; q.Gr = d.Gr; q.Gw = d.Gw;
    q.K = (long long)pr.B * pr.T;
    const int mt = (d.Gr * pr.D + DR_M - 1) / DR_M, pt = (pr.D + DR_P - 1) / DR_P;
    long long splits = 592 / ((long long)mt * pt * pr.N);  // about four CTAs per SM
    if (splits < 1) splits = 1;
    if (splits > (q.K + 127) / 128) splits = (q.K + 127) / 128;
    if ((long long)pr.N * splits > 65535) splits = 65535 / pr.N;
    q.rows_per_split = (int)(((q.K + splits - 1) / splits + DR_K - 1) / DR_K * DR_K);
    splits = (q.K + q.rows_per_split - 1) / q.rows_per_split;
    x32_dr_kernel<<<dim3((unsigned)mt, (unsigned)pt, (unsigned)(pr.N * splits)), XTHREADS, 0, stream>>>(q);
    e = cudaGetLastError();
  }
  return (int)e;
}

__attribute__((visibility("hidden"))) int frnn_finalize_grads_f32(const frnn_plan* plan, const void* grads_f32, void* dR, void* db, void* stream_) {
  Dims d;
  Tile tl;
  int rc = check(plan, &d, &tl);
  if (rc) return rc;
  if (!grads_f32 || !dR || !db) return FRNN_ERR_NULL;
  const frnn_problem& pr = plan->prob;
  const size_t nR = (size_t)d.Gr * pr.N * pr.D * pr.D, nb = (size_t)d.Gt * pr.N * pr.D;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemcpyAsync(dR, grads_f32, nR * 4, cudaMemcpyDeviceToDevice, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyAsync(db, static_cast<const float*>(grads_f32) + nR, nb * 4, cudaMemcpyDeviceToDevice, stream);
}

}  // extern "C"
#endif  // FRNN_F16
