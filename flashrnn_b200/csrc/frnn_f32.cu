// float32 kernel dtype: Wx, R, b, the states and every gradient are fp32 and so is all arithmetic.
//
// The reference offers dtype="float32" for every cell (tests/test_lstm.py:48-60; its fused kernel then multiplies in
// tf32, fused/flashrnn_fused_forward.cu:108-112).  Here the fp32 path is the ACCURATE one: products and sums in fp32 on
// the CUDA cores, gate nonlinearities from exp (error ~1e-6), so that it agrees with the fp32 `vanilla` loop to ~1e-5 --
// the 16-bit tensor-core loops are the fast path, this one is for callers that need float32 results (reference checks,
// gradient checks, small models).  Same structure as the other loops, kept simple:
//   * forward: one CTA per (head, 8 batch rows) runs all T steps.  Per step: pre = R h_{t-1} (thread = gate row, R read
//     transposed so that a warp reads consecutive addresses, from shared memory when the head's R fits there, else from
//     L2; h broadcast from shared memory), then the pointwise cell on (row, unit) items, new h into the shared tile.
//   * backward: the reverse loop with the closed-form cell backward; dh_{t-1} = R^T delta (thread = input unit p);
//     the carried cotangents live in the ds0 output itself, db is summed in shared memory and flushed once.
//   * dR: a tiled fp32 GEMM over all (b, t) with split-K and fp32 atomics.
// Replaces, for float32, FLASHRNNCellFusedForward / FLASHRNNCellFusedBackward / the cuBLAS dR GEMM of the reference
// (fused/flashrnn_fused_forward.cu:146-659, fused/flashrnn_fused_backward.cu:129-624, 1049-1058).
#ifndef FRNN_F16  // compiled once, into the bfloat16 build, which owns the public entry points
#define FRNN_NS_OVERRIDE frnn_x32
#define FRNN_EXACT_ACT 1
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
  int B, T, N, D;
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

// dR[g][n][d][p] += sum over this CTA's rows k = (b, t) of delta_g[k][d] * h_{t-1}[k][p]: 64 x 64 tile of ((g, d), p)
struct XDrParams {
  const float* dWx; const float* dg0; const float* states; const float* s0; float* dR;
  int cell, B, T, N, D, Gr, Gw;
  long long K;
  int rows_per_split;
};
__global__ void __launch_bounds__(XTHREADS) x32_dr_kernel(const XDrParams p) {
  __shared__ float As[32][65], Hs[32][65];
  const int D = p.D, N = p.N, T = p.T, GD = p.Gr * D;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * 64, p0 = blockIdx.y * 64;
  const int n = blockIdx.z % N, split = blockIdx.z / N;
  const size_t ND = (size_t)N * D;
  const long long k0 = (long long)split * p.rows_per_split;
  long long k1 = k0 + p.rows_per_split;
  if (k1 > p.K) k1 = p.K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (long long kc = k0; kc < k1; kc += 32) {
    for (int i = tid; i < 32 * 64; i += XTHREADS) {
      const int kk = i >> 6, c = i & 63;
      const long long k = kc + kk;
      float a = 0.f, hv = 0.f;
      if (k < k1) {
        const long long b = k / T;
        const int t = (int)(k - b * T);
        const int m = m0 + c;
        if (m < GD) {
          const int g = m / D, d = m - g * D;
          if (p.cell == CELL_GRU && g == 0) a = p.dg0[(size_t)k * ND + (size_t)n * D + d];
          else a = p.dWx[((size_t)k * p.Gw + (p.cell == CELL_GRU ? g - 1 : g)) * ND + (size_t)n * D + d];
        }
        const int pc = p0 + c;
        if (pc < D) hv = t > 0 ? p.states[(size_t)(k - 1) * ND + (size_t)n * D + pc] : p.s0[(size_t)b * ND + (size_t)n * D + pc];
      }
      As[kk][c] = a;
      Hs[kk][c] = hv;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      float a[4], hh[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; hh[i] = Hs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], hh[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
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
int validate(const frnn_problem* pr, Dims* d) {
  if (!pr) return FRNN_ERR_NULL;
  if (!dims_of(pr->cell, pr->forward_clip, d)) return FRNN_ERR_CELL;
  if (pr->dtype_io != FRNN_DTYPE_F32 || pr->dtype_state != FRNN_DTYPE_F32) return FRNN_ERR_DTYPE;
  if (pr->B < 1 || pr->T < 1 || pr->N < 1 || pr->N > 65535 || pr->D < 4 || pr->D > 1024 || pr->D % 4) return FRNN_ERR_SHAPE;
  if ((pr->B + XBT - 1) / XBT > 65535) return FRNN_ERR_SHAPE;
  if (fwd_smem(*pr, *d, false) > kSmemMax || bwd_smem(*pr, *d) > kSmemMax) return FRNN_ERR_SHAPE;
  return FRNN_OK;
}
int check(const frnn_plan* pl, Dims* d) {
  if (!pl) return FRNN_ERR_NULL;
  if (pl->abi_version != FRNN_ABI_VERSION) return FRNN_ERR_PLAN;
  const int rc = validate(&pl->prob, d);
  if (rc) return rc;
  if (pl->cluster_size != 1 || pl->batch_tile != XBT || pl->threads != XTHREADS || pl->units_per_cta != pl->prob.D ||
      pl->workspace_bytes != ws_layout(pl->prob, *d).total || pl->probe_noop_cell)
    return FRNN_ERR_PLAN;
  return FRNN_OK;
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
  if ((cs && cs != 1) || (bt && bt != XBT) || stages) return FRNN_ERR_PLAN;  // the float32 loops have one geometry
  frnn_plan pl = {};
  pl.abi_version = FRNN_ABI_VERSION;
  pl.prob = *pr;
  pl.cluster_size = 1;
  pl.units_per_cta = pr->D;
  pl.batch_tile = XBT;
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
  int rc = check(plan, &d);
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
  p.r_in_smem = fwd_smem(pr, d, true) <= kSmemMax;
  p.fclip = pr.forward_clip; p.gclip = pr.grad_clip; p.grad_cut = pr.grad_cut;
  p.wx_sb = wxs[0]; p.wx_st = wxs[1]; p.wx_sg = wxs[2]; p.wx_sn = wxs[3];
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
  int rc = check(plan, &d);
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
    if (e != cudaSuccess) return (int)e;
  }
  if (parts & FRNN_PART_DR) {
    XDrParams q = {};
    q.dWx = static_cast<const float*>(a->dWx); q.dg0 = reinterpret_cast<const float*>(ws + w.dg0);
    q.states = static_cast<const float*>(a->states); q.s0 = static_cast<const float*>(a->s0); q.dR = grads;
    q.cell = pr.cell; q.B = pr.B; q.T = pr.T; q.N = pr.N; q.D = pr.D; q.Gr = d.Gr; q.Gw = d.Gw;
    q.K = (long long)pr.B * pr.T;
    const int mt = (d.Gr * pr.D + 63) / 64, pt = (pr.D + 63) / 64;
    long long splits = 592 / ((long long)mt * pt * pr.N);  // about four CTAs per SM
    if (splits < 1) splits = 1;
    if (splits > (q.K + 127) / 128) splits = (q.K + 127) / 128;
    if ((long long)pr.N * splits > 65535) splits = 65535 / pr.N;
    q.rows_per_split = (int)(((q.K + splits - 1) / splits + 31) / 32 * 32);
    splits = (q.K + q.rows_per_split - 1) / q.rows_per_split;
    x32_dr_kernel<<<dim3((unsigned)mt, (unsigned)pt, (unsigned)(pr.N * splits)), XTHREADS, 0, stream>>>(q);
    e = cudaGetLastError();
  }
  return (int)e;
}

__attribute__((visibility("hidden"))) int frnn_finalize_grads_f32(const frnn_plan* plan, const void* grads_f32, void* dR, void* db, void* stream_) {
  Dims d;
  int rc = check(plan, &d);
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
