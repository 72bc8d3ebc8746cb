// Backward time loop (reverse recurrence), one persistent launch for all T steps.
//
// Same work split as the forward kernel: a cluster of CS CTAs owns one (head, batch tile); CTA c owns
// hidden units [c*U, (c+1)*U).  It keeps the TRANSPOSED slice R^T[p in its units][all Gr*D gate rows] in
// registers as warp-MMA A fragments: warp (g, ug) holds the columns of gate g for 16 of its units.
// Per step t = T-1 .. 0
//   phase B  every thread owns fixed (unit pair, batch row) items: total dh = external cotangent +
//            recurrent part (sum of the Gr partial products left in shared memory by phase A of the
//            previous iteration, optionally clipped); closed-form cell backward in fp32 gives the gate
//            deltas; the deltas of the R-connected gates go (bf16) into this CTA's slice of the delta
//            buffer; dWx goes to global memory; db and the carried cotangents (dc, dn, GRU's z*dh) stay
//            in registers;
//   push     one thread per peer CTA starts a bulk async copy of the slice into the peer's delta buffer,
//            completing on the peer's mbarrier (no cluster barrier, no fence);
//   wait     for the slices of the other CTAs (bounded mbarrier wait);
//   phase A  dh_{t-1}[p] partials = R^T slice x deltas (BT x Gr*D) on the tensor cores -> shared memory.
//
// Two ways to organise the cross-CTA part of dh_{t-1} = R^T delta (template parameter MPW):
//   MPW == 0  "all-gather": every CTA receives the deltas of all CTAs (bf16, Gr*U values per row and CTA) and
//             multiplies them with its rows p of R^T.  Works for every cluster size.
//   MPW  > 0  "reduce-scatter": every CTA multiplies ONLY ITS OWN deltas with all D rows of R^T restricted to its
//             columns (each warp: MPW row tiles x all local k-steps) right after phase B -- no wait in between --
//             and sends each peer the fp32 partial sums of that peer's rows; the owner adds the CS partials in its
//             next phase B.  A cluster moves 2-4x fewer bytes per step this way (the exchange is bound by the
//             ~120 B/clk a cluster's shared-memory network sustains).  Needs CS == MPW * Gr.
// Cache / state / cotangent values are prefetched kStages steps ahead with cp.async.
//
// Replaces FLASHRNNCellFusedBackward (reference flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:129-624),
// the FLASHRNNPointwiseBackward functions (fused/*_fused_pointwise.cuh; GRU: alternating/gru_pointwise.cu:120-193)
// and gradientBiasAggregationKernel (flashrnn_fused_backward.cu:626-665).
#pragma once
#include "frnn_common.cuh"

namespace FRNN_NS {

// Closed-form backward of one cell update, fp32.
//   dh        total cotangent of h_t (external + recurrent)
//   dext[k]   external cotangents of the states 1..NEXT-1 (dext[0] unused)
//   car[s]    in: cotangent carried from step t+1 for state s (s >= 1); out: carried to step t-1.
//             car[0] out = the direct (non-matrix) part of dh_{t-1} (GRU: z * dh), else 0.
//   cur[k]/prv[k]  needed states (Cell::need(k)) at t and t-1
//   dR_[g]    deltas of the R-connected gates (order of R), dW_[g] of the Wx gates, dB_[g] of the bias gates
template <int CELL>
__device__ __forceinline__ void cell_backward(float dh, const float* dext, float* car, const float* cache,
                                              const float* cur, const float* prv, float* dR_, float* dW_,
                                              float* dB_) {
  if constexpr ((CELL & kNoopCell) != 0) {  // chain-floor probe: no gate math
    using C = Cell<CELL>;
    const float dg = 0.25f * dh + cache[0] * 0.f;
#pragma unroll
    for (int g = 0; g < C::Gr; ++g) dR_[g] = dg;
#pragma unroll
    for (int g = 0; g < C::Gw; ++g) dW_[g] = dg;
#pragma unroll
    for (int g = 0; g < C::Gt; ++g) dB_[g] = dg;
#pragma unroll
    for (int s = 0; s < C::S; ++s) car[s] = 0.f;
  } else if constexpr (CELL == CELL_LSTM) {  // vanilla_fwbw/bw.py:100-133
    const float ig = cache[0], fg = cache[1], zv = cache[2], og = cache[3];
    const float tc = fast_tanh(cur[0]);
    const float dc = dext[1] + car[1] + dh * og * (1.f - tc * tc);
    dR_[0] = dc * zv * ig * (1.f - ig);
    dR_[1] = dc * prv[0] * fg * (1.f - fg);
    dR_[2] = dc * ig * (1.f - zv * zv);
    dR_[3] = dh * tc * og * (1.f - og);
#pragma unroll
    for (int g = 0; g < 4; ++g) { dW_[g] = dR_[g]; dB_[g] = dR_[g]; }
    car[0] = 0.f; car[1] = dc * fg;
  } else if constexpr (CELL == CELL_GRU) {  // alternating/gru_pointwise.cu:120-193
    const float gr = cache[0], rg = cache[1], zg = cache[2], nv = cache[3];
    const float dz = dh * (prv[0] - nv) * zg * (1.f - zg);
    const float dn = dh * (1.f - zg) * (1.f - nv * nv);
    const float dr = dn * gr * rg * (1.f - rg);
    const float dg = dn * rg;
    dR_[0] = dg; dR_[1] = dr; dR_[2] = dz;
    dW_[0] = dr; dW_[1] = dz; dW_[2] = dn;
    dB_[0] = dg; dB_[1] = dr; dB_[2] = dz; dB_[3] = dn;
    car[0] = zg * dh;
  } else if constexpr (CELL == CELL_ELMAN || CELL == CELL_ELMAN_CLIP) {  // fused/elman_fused_pointwise.cuh:62-93
    const float hv = (CELL == CELL_ELMAN_CLIP) ? cache[0] : cur[0];  // the tanh output (before any forward clamp)
    const float dg = dh * (1.f - hv * hv);
    dR_[0] = dg; dW_[0] = dg; dB_[0] = dg;
    car[0] = 0.f;
  } else {  // sLSTM, vanilla_fwbw/bw.py:136-189 (stabiliser m treated as a constant)
    const float ig = cache[0], fg = cache[1], zv = cache[2], og = cache[3], omsf = cache[4];
    const float cn = cur[0], n2 = cur[1];
    const float inv_n = __fdividef(1.f, n2);
    const float dc = dext[1] + car[1] + dh * og * inv_n;
    const float dn = dext[2] + car[2] - dh * og * cn * inv_n * inv_n;
    dR_[0] = ig * (zv * dc + dn);
    dR_[1] = fg * (dc * prv[0] + dn * prv[1]) * omsf;
    dR_[2] = dc * ig * (1.f - zv * zv);
    dR_[3] = dh * cn * inv_n * og * (1.f - og);
#pragma unroll
    for (int g = 0; g < 4; ++g) { dW_[g] = dR_[g]; dB_[g] = dR_[g]; }
    car[0] = 0.f; car[1] = fg * dc; car[2] = fg * dn; car[3] = 0.f;
  }
}

// U and CS implied by a reduce-scatter instantiation: all Gr*U/16 local k-steps per warp, MPW row tiles per warp
template <int CELL, int KT, int MPW> struct RsGeom {
  static constexpr int KPW = MPW > 0 ? KT / MPW : 0;              // local k-steps = Gr * U / 16
  static constexpr int NUT = MPW > 0 ? KPW / Cell<CELL>::Gr : 0;  // 16-unit tiles per CTA
  static constexpr int U = NUT * 16;
  static constexpr int CS = MPW * Cell<CELL>::Gr;
  static constexpr bool valid = MPW > 0 && KT % MPW == 0 && KPW % Cell<CELL>::Gr == 0 && NUT >= 1 &&
                                (NUT & (NUT - 1)) == 0 && CS <= 16 && CS * U == KT * 16;
};

template <int CELL, int NT, int MPW>
__host__ __device__ constexpr size_t bwd_smem_bytes(int D, int U, int threads) {
  using C = Cell<CELL>;
  constexpr int BT = NT * 8;
  constexpr int IPT = (BT + 4 * C::Gr - 1) / (4 * C::Gr);
  constexpr int GCA = C::GC > 0 ? C::GC : 1;
  const int CS = D / U;
  const size_t rl = ring_row_len(U, BT, threads);
  const size_t rings = (size_t)kStages * GCA * IPT * rl * 4 + (size_t)kStages * (C::NNEED + C::NEXT) * IPT * rl * 8 + 32;
  if (MPW > 0)  // delta tile + double-buffered send and receive slices of fp32 partials
    return (size_t)BT * (C::Gr * U + 8) * 2 + (size_t)4 * CS * BT * (U + 4) * 4 + rings;
  return (size_t)2 * CS * BT * (C::Gr * U + 8) * 2 + (size_t)C::Gr * BT * (U + 4) * 4 + rings;
}

// KT / DYN as in the forward kernel: KT k-steps of R^T per warp stay in registers; with DYN the head dim is a run-time
// value above 256 and the remaining k-steps are streamed from global memory every step (all-gather form only).
template <int CELL, int KT, int NT, int MPW, bool DYN>
__global__ void __launch_bounds__(LaunchBounds<CELL, KT>::threads, LaunchBounds<CELL, KT>::min_blocks) frnn_bwd_kernel(const __grid_constant__ LoopParams p) {
  using C = Cell<CELL>;
  static_assert(!(DYN && MPW > 0), "the streamed form exists for the all-gather exchange only");
  constexpr int Gr = C::Gr, Gw = C::Gw, Gt = C::Gt, S = C::S, GC = C::GC, NNEED = C::NNEED, NEXT = C::NEXT;
  constexpr int BT = NT * 8;
  const int D = DYN ? p.D : KT * 16;
  const int ktot = DYN ? (p.D >> 4) : KT;  // k-steps per gate in a row of R^T
  constexpr int IPT = (BT + 4 * Gr - 1) / (4 * Gr);
  constexpr int GCA = GC > 0 ? GC : 1;
  constexpr int NSS = NNEED + NEXT;  // 8-byte slots per item and stage in the state ring
  constexpr bool RS = MPW > 0;
  constexpr int KPW = RS ? KT / (RS ? MPW : 1) : KT;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x;
  const int U = p.U, CS = p.CS, T = p.T, N = p.N, B = p.B;
  const int GS = Gr * U + 8;        // row pitch (elements) of a delta tile: [b][g*U + u]
  const int SL = BT * GS;           // elements per delta slice
  const int ushift = 31 - __clz(U >> 4);
  const int PS = U + 4;             // row pitch (floats) of a partial-sum tile [b][u]; == 4 (mod 16): conflict-free stores
  const int PSL = BT * PS;          // floats per partial-sum slice
  const int n = blockIdx.z, bt0 = blockIdx.y * BT;
  const uint32_t crank = (CS > 1) ? cluster_ctarank() : 0u;
  const int unit0 = (int)crank * U;
  const size_t ND = (size_t)N * D;
  const int f32 = p.state_f32;
  const int nUT = U >> 4;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  // all-gather:      dgbuf [2][CS][BT][GS] bf16 | part [Gr][BT][PS] f32
  // reduce-scatter:  dgbuf [BT][GS] bf16        | stage [2][CS][BT][PS] f32 | recv [2][CS][BT][PS] f32
  elem_t* dgbuf = reinterpret_cast<elem_t*>(smem_raw);
  float* part = reinterpret_cast<float*>(smem_raw + (RS ? (size_t)SL * 2 : (size_t)2 * CS * SL * 2));
  float* stage_buf = part;                                  // RS only
  float* recv_buf = part + (size_t)2 * CS * PSL;            // RS only
  uint32_t* ringc = reinterpret_cast<uint32_t*>(part + (RS ? (size_t)4 * CS * PSL : (size_t)Gr * BT * PS));  // [kStages][GCA][IPT][nthr]
  const int RL = ring_row_len(U, BT, nthr);  // threads that own items: the rings have one slot row per such thread
  uint2* rings = reinterpret_cast<uint2*>(ringc + (size_t)kStages * GCA * IPT * RL);    // [kStages][NSS][IPT][RL]
  uint64_t* full = reinterpret_cast<uint64_t*>(rings + (size_t)kStages * NSS * IPT * RL);  // [2]
  // gave_up[j & 1] is set by a thread whose bounded wait expired in step index j
  volatile int* gave_up = reinterpret_cast<volatile int*>(full + 2);

  // ---- this warp's fragments of R^T (rows p, columns = gate rows), resident for the whole sequence
  const int g_w = warp / nUT, ug_w = warp - g_w * nUT;  // all-gather: gate / unit tile of this warp
  uint4 Rreg[KT];
  const uint4* rsrc = p.Rpack + ((((size_t)n * Gr + g_w) * ktot + (unit0 / 16 + ug_w)) * ktot) * 32 + lane;  // all-gather row
  if constexpr (RS) {
    // rows p: tiles warp*MPW + mi (all D rows are covered by the CTA's warps); columns: the CTA's own (g, u)
#pragma unroll
    for (int mi = 0; mi < MPW; ++mi)
#pragma unroll
      for (int ks = 0; ks < KPW; ++ks) {
        const int g = ks / nUT, ul = ks - g * nUT;
        Rreg[mi * KPW + ks] = __ldg(p.Rpack + ((((size_t)n * Gr + g) * ktot + (warp * MPW + mi)) * ktot + (unit0 / 16 + ul)) * 32 + lane);
      }
  } else {
#pragma unroll
    for (int k = 0; k < KT; ++k) Rreg[k] = __ldg(rsrc + k * 32);
  }

  // ---- items
  const int half_u = U >> 1, nitems = half_u * BT;
  const size_t cta_lin = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  const size_t st_esz = f32 ? 4 : 2;
  const size_t st_sstride = (size_t)B * T * ND * st_esz;
  const size_t ch_step = (size_t)gridDim.x * gridDim.y * gridDim.z * GCA * nitems;
  bool it_on[IPT], it_ok[IPT];
  uint32_t part_it[IPT];                // float offset of (bl, 2*up) inside a partial-sum tile
  uint32_t dloc_it[IPT];                // element offset of (bl, gate 0, 2*up) inside a delta tile
  const uint32_t* ch_pf[IPT];           // cache of the next step to prefetch
  const unsigned char* st_pf[IPT];      // states[0][b][t-1] of the next step to prefetch
  const unsigned char* ds_pf[IPT];      // dstates[0][b][t]  of the next step to prefetch
  const unsigned char* s0_it[IPT];      // s0[0][b]
  elem_t* dwx_ptr[IPT];          // dWx[b][t][0][n][d] of the current step
  elem_t* dg0_ptr[IPT];
  size_t s0_off[IPT];
  float car[IPT][S][2], cur[IPT][NNEED][2], dbacc[IPT][Gt][2];
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int q = tid + i * nthr;
    it_on[i] = q < nitems;
    const int bl = it_on[i] ? q / half_u : 0, up = it_on[i] ? q - bl * half_u : 0;
    const int bg = bt0 + bl, d = unit0 + 2 * up;
    it_ok[i] = it_on[i] && bg < B;
    const int bgc = bg < B ? bg : B - 1;
    part_it[i] = (uint32_t)(bl * PS + 2 * up);
    dloc_it[i] = (uint32_t)(bl * GS + 2 * up);
    const size_t st_off = ((size_t)bgc * T) * ND + (size_t)n * D + d;
    s0_off[i] = ((size_t)bgc) * ND + (size_t)n * D + d;  // + s*B*ND
    ch_pf[i] = reinterpret_cast<const uint32_t*>(p.cache) + cta_lin * GCA * nitems + (it_on[i] ? q : 0) + (size_t)(T - 1) * ch_step;
    st_pf[i] = static_cast<const unsigned char*>(p.states) + (st_off + (size_t)(T - 2) * ND) * st_esz;  // valid for T >= 2
    ds_pf[i] = static_cast<const unsigned char*>(p.dstates) +
               ((size_t)bgc * p.ds_sb + (size_t)(T - 1) * p.ds_st + (size_t)n * p.ds_sn + d) * st_esz;
    s0_it[i] = static_cast<const unsigned char*>(p.s0) + s0_off[i] * st_esz;
    dwx_ptr[i] = p.dWx + ((size_t)bgc * T * Gw) * ND + (size_t)n * D + d + (size_t)(T - 1) * Gw * ND;
    dg0_ptr[i] = p.dg0 + st_off + (size_t)(T - 1) * ND;
#pragma unroll
    for (int s = 0; s < S; ++s) { car[i][s][0] = 0.f; car[i][s][1] = 0.f; }
#pragma unroll
    for (int g = 0; g < Gt; ++g) { dbacc[i][g][0] = 0.f; dbacc[i][g][1] = 0.f; }
#pragma unroll
    for (int k = 0; k < NNEED; ++k) {
      float2 v = make_float2(0.f, 0.f);
      if (it_ok[i]) v = load_state2(p.states, st_off + ((size_t)C::need(k) * B * T + (T - 1)) * ND, f32);
      cur[i][k][0] = v.x; cur[i][k][1] = v.y;
    }
  }
  // no recurrent cotangent flows into the last time step: the partial sums read by the first phase B are zero
  for (int idx = tid; idx < (RS ? 4 * CS * PSL : Gr * BT * PS); idx += nthr) part[idx] = 0.f;

  // ---- prefetch ring: everything step t needs except what is carried in registers.  Issued in step order
  // T-1, T-2, ...; `t` is the step being prefetched.
  auto issue = [&](int t, int stage) {
    if (t >= 0) {
#pragma unroll
      for (int i = 0; i < IPT; ++i) {
        if (!it_ok[i]) continue;
#pragma unroll
        for (int k = 0; k < GC; ++k)
          cp_async4(ringc + ((size_t)(stage * GCA + k) * IPT + i) * RL + tid, ch_pf[i] + (size_t)k * nitems);
        ch_pf[i] -= ch_step;
#pragma unroll
        for (int k = 0; k < NNEED; ++k) {  // state at t-1 (initial state for t == 0)
          uint2* dst = rings + ((size_t)(stage * NSS + k) * IPT + i) * RL + tid;
          const unsigned char* src = (t > 0) ? st_pf[i] + (size_t)C::need(k) * st_sstride
                                             : s0_it[i] + (size_t)C::need(k) * B * ND * st_esz;
          if (f32) cp_async8(dst, src); else cp_async4(dst, src);
        }
#pragma unroll
        for (int k = 0; k < NEXT; ++k) {  // external cotangent of state k at t
          uint2* dst = rings + ((size_t)(stage * NSS + NNEED + k) * IPT + i) * RL + tid;
          const unsigned char* src = ds_pf[i] + (size_t)k * p.ds_ss * st_esz;
          if (f32) cp_async8(dst, src); else cp_async4(dst, src);
        }
        st_pf[i] -= ND * st_esz;
        ds_pf[i] -= (size_t)p.ds_st * st_esz;
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < IPT; ++i)
    if (it_on[i] && !it_ok[i])  // rows beyond B: their inputs read as zero
      for (int s = 0; s < kStages; ++s) {
#pragma unroll
        for (int k = 0; k < GCA; ++k) ringc[((size_t)(s * GCA + k) * IPT + i) * RL + tid] = 0u;
#pragma unroll
        for (int k = 0; k < NSS; ++k) rings[((size_t)(s * NSS + k) * IPT + i) * RL + tid] = make_uint2(0u, 0u);
      }
#pragma unroll
  for (int s = 0; s < kStages; ++s) issue(T - 1 - s, s);

  // ---- cluster set-up.  full[x] counts the bytes delivered into buffer x (x = step index & 1)
  const uint32_t slice_bytes = RS ? (uint32_t)(PSL * 4) : (uint32_t)(SL * 2);
  const uint32_t expect_bytes = (uint32_t)(CS - 1) * slice_bytes;
  bool poisoned = false;
  if (CS > 1) {
    if (tid == 0) {
      gave_up[0] = 0;
      gave_up[1] = 0;
      mbar_init(&full[0], 1);
      mbar_init(&full[1], 1);
      fence_mbar_init();
      mbar_arrive_expect_tx(&full[0], expect_bytes);             // exchange of step index 0 (t = T-1)
      if (T > 1) mbar_arrive_expect_tx(&full[1], expect_bytes);  // step index 1
    }
    cluster_arrive();
    cluster_wait();
  } else {
    __syncthreads();
  }
  const uint32_t full_u32 = smem_u32(&full[0]);
  auto ring_state = [&](int stage, int slot, int i) -> float2 {
    const uint2 w = rings[((size_t)(stage * NSS + slot) * IPT + i) * RL + tid];
    if (f32) return make_float2(__uint_as_float(w.x), __uint_as_float(w.y));
    return unpack_x2(w.x);
  };
  // recurrent part of dh for item i: sum of the partial products of the previous step (`pbuf` = its buffer index)
  auto recurrent_sum = [&](int i, int pbuf, float (&rec)[2]) {
    if constexpr (RS) {
      // the cluster size of this exchange scheme is a constant of the instantiation: all loads are issued before the
      // first addition, and the additions form two short chains instead of one of CS links
      constexpr int CSC = (RS ? MPW : 1) * Gr;
      const float* src = recv_buf + (size_t)pbuf * CSC * PSL + part_it[i];
      float2 v[CSC];
#pragma unroll
      for (int c = 0; c < CSC; ++c) v[c] = *reinterpret_cast<const float2*>(src + (size_t)c * PSL);
      float ax = 0.f, ay = 0.f, bx = 0.f, by = 0.f;
#pragma unroll
      for (int c = 0; c < CSC; c += 2) {
        ax += v[c].x; ay += v[c].y;
        if (c + 1 < CSC) { bx += v[c + 1].x; by += v[c + 1].y; }
      }
      rec[0] += ax + bx; rec[1] += ay + by;
    } else {
#pragma unroll
      for (int g = 0; g < Gr; ++g) {
        const float2 v = *reinterpret_cast<const float2*>(part + (size_t)g * BT * PS + part_it[i]);
        rec[0] += v.x; rec[1] += v.y;
      }
    }
  };
  // data of step index j has landed in buffer `buf`; `slot` = parity of the step index the wait happens in
  auto wait_exchange = [&](int buf, int j, int t, int slot) {
    if (CS > 1) {
      if (!poisoned && !mbar_wait_bounded(&full[buf], (uint32_t)((j >> 1) & 1))) {
        poisoned = true;
        gave_up[slot] = 1;
        report_timeout(p.status, t);
      }
      // re-arm for step index j + 2; never after an expired wait: that phase is still open, no arrival left to give
      if (tid == 0 && !poisoned && j + 2 < T) mbar_arrive_expect_tx(&full[buf], expect_bytes);
    }
  };

  int stage = 0;
  for (int j = 0; j < T; ++j) {  // j-th step of the reverse loop, time index t = T-1-j
    const int t = T - 1 - j, buf = j & 1;
    cp_async_wait<kStages - 1>();
    if constexpr (RS) { if (j > 0) wait_exchange(buf ^ 1, j - 1, t, buf); }  // partial sums produced in step j-1
    float dwv[IPT][Gw][2], dg0v[IPT][2];
    elem_t* ddst = RS ? dgbuf : dgbuf + (size_t)buf * CS * SL + (size_t)crank * SL;
    // ---------------- phase B: pointwise backward; R-gate deltas (bf16) into the delta tile
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_on[i]) continue;
      float rec[2] = {car[i][0][0], car[i][0][1]};
      if (!p.grad_cut) recurrent_sum(i, buf ^ 1, rec);
      float prvv[NNEED][2], extv[NEXT][2], chv[GCA][2];
#pragma unroll
      for (int k = 0; k < NNEED; ++k) { const float2 v = ring_state(stage, k, i); prvv[k][0] = v.x; prvv[k][1] = v.y; }
#pragma unroll
      for (int k = 0; k < NEXT; ++k) { const float2 v = ring_state(stage, NNEED + k, i); extv[k][0] = v.x; extv[k][1] = v.y; }
#pragma unroll
      for (int k = 0; k < GC; ++k) {
        const float2 v = unpack_x2(ringc[((size_t)(stage * GCA + k) * IPT + i) * RL + tid]);
        chv[k][0] = v.x; chv[k][1] = v.y;
      }
      float dRv[2][Gr];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float r = rec[e];
        if (p.gclip > 0.f) r = clampf(r, p.gclip);
        float dext[NEXT], cr[S], cc[GCA], cu[NNEED], pv[NNEED], dW_[Gw], dB_[Gt];
#pragma unroll
        for (int k = 0; k < NEXT; ++k) dext[k] = extv[k][e];
#pragma unroll
        for (int s = 0; s < S; ++s) cr[s] = car[i][s][e];
#pragma unroll
        for (int k = 0; k < GC; ++k) cc[k] = chv[k][e];
#pragma unroll
        for (int k = 0; k < NNEED; ++k) { cu[k] = cur[i][k][e]; pv[k] = prvv[k][e]; }
        cell_backward<CELL>(dext[0] + r, dext, cr, cc, cu, pv, dRv[e], dW_, dB_);
#pragma unroll
        for (int s = 0; s < S; ++s) car[i][s][e] = it_ok[i] ? cr[s] : 0.f;
#pragma unroll
        for (int g = 0; g < Gw; ++g) dwv[i][g][e] = dW_[g];
#pragma unroll
        for (int g = 0; g < Gt; ++g) dbacc[i][g][e] += it_ok[i] ? dB_[g] : 0.f;
        if (!it_ok[i]) {
#pragma unroll
          for (int g = 0; g < Gr; ++g) dRv[e][g] = 0.f;
        }
#pragma unroll
        for (int k = 0; k < NNEED; ++k) cur[i][k][e] = pv[k];
      }
      dg0v[i][0] = dRv[0][0]; dg0v[i][1] = dRv[1][0];
#pragma unroll
      for (int g = 0; g < Gr; ++g)
        *reinterpret_cast<uint32_t*>(ddst + dloc_it[i] + g * U) = pack_x2(dRv[0][g], dRv[1][g]);
    }
    if (!RS && CS > 1) fence_proxy_async_smem();
    __syncthreads();
    // Set when a wait expired in some thread of this CTA: in this step before the barrier above (reduce-scatter), or in
    // the previous step (all-gather, whose wait follows this barrier).  Either way the write precedes the barrier and
    // no thread writes this slot again before the next one, so every thread reads the same value.  The CTA acts on
    // it at the end of the step, where the load has long landed.
    const int quit = (CS > 1) ? gave_up[RS ? buf : buf ^ 1] : 0;
    if constexpr (RS) {
      // ---------------- phase A (reduce-scatter): partial dh_{t-1}[all p] from this CTA's deltas only
      float* sbuf = stage_buf + (size_t)buf * CS * PSL;
      float* rbuf = recv_buf + (size_t)buf * CS * PSL;
      const int gid = lane >> 2, tig = lane & 3;
      float acc[RS ? MPW : 1][NT][4];
      warp_mma_tiles<(RS ? MPW : 1), KPW, NT>(Rreg, dgbuf, GS, lane, acc);
#pragma unroll
      for (int mi = 0; mi < MPW; ++mi) {
        const int mt = warp * MPW + mi;                 // row tile of p: owner CTA = mt / nUT
        const int dest = mt >> ushift, ul = mt & (nUT - 1);
        float* dst = ((uint32_t)dest == crank ? rbuf : sbuf) + (size_t)dest * PSL + ul * 16 + gid;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int b0 = nt * 8 + 2 * tig;
          dst[(size_t)b0 * PS] = acc[mi][nt][0];
          dst[(size_t)(b0 + 1) * PS] = acc[mi][nt][1];
          dst[(size_t)b0 * PS + 8] = acc[mi][nt][2];
          dst[(size_t)(b0 + 1) * PS + 8] = acc[mi][nt][3];
        }
      }
      if (CS > 1) fence_proxy_async_smem();
      __syncthreads();
      // ---------------- push the partial sums of every peer's rows into that peer's receive slice [buf][me]
      if (CS > 1 && !(p.test_drop && crank == 0 && j == 0)) {  // (test hook: CTA 0 may withhold its first message)
        __syncwarp();
        const uint32_t s0a = smem_u32(sbuf), r0a = smem_u32(rbuf) + crank * slice_bytes;
#pragma unroll 1
        for (uint32_t c = (uint32_t)warp; c < (uint32_t)CS; c += (uint32_t)(nthr >> 5)) {
          if (c == crank) continue;
          const uint32_t dsta = map_to_cta(r0a, c), bara = map_to_cta(full_u32 + buf * 8, c);
          if (elect_one_sync()) bulk_copy_to_cta(dsta, s0a + c * slice_bytes, slice_bytes, bara);
        }
      }
    } else {
      // ---------------- push this CTA's delta slice to every other CTA of the cluster
      if (CS > 1 && !(p.test_drop && crank == 0 && j == 0))  // uniform branch; one elected lane per warp copies
        push_slice_to_peers(smem_u32(ddst), slice_bytes, full_u32 + buf * 8, crank, (uint32_t)CS, (uint32_t)warp,
                            (uint32_t)(nthr >> 5));
    }
    // ---------------- off the critical path: dWx to global memory, next prefetch
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_ok[i]) continue;
#pragma unroll
      for (int g = 0; g < Gw; ++g)
        *reinterpret_cast<uint32_t*>(dwx_ptr[i] + (size_t)g * ND) = pack_x2(dwv[i][g][0], dwv[i][g][1]);
      dwx_ptr[i] -= (size_t)Gw * ND;
      if (CELL == CELL_GRU) {
        *reinterpret_cast<uint32_t*>(dg0_ptr[i]) = pack_x2(dg0v[i][0], dg0v[i][1]);
        dg0_ptr[i] -= ND;
      }
    }
    issue(t - kStages, stage);
    stage = (stage + 1 == kStages) ? 0 : stage + 1;
    if constexpr (!RS) {
      wait_exchange(buf, j, t, buf);
      // ---------------- phase A (all-gather): part[g][b][p] = sum_d R[g][d][p] * delta_g[b][d]
      float acc[NT][4];
      warp_mma_rows<KT, NT>(Rreg, dgbuf + (size_t)buf * CS * SL, GS, g_w * U, ushift, SL, lane, acc);
      if constexpr (DYN) warp_mma_stream<NT>(rsrc, KT, ktot, dgbuf + (size_t)buf * CS * SL, GS, g_w * U, ushift, SL, lane, acc);
      const int gid = lane >> 2, tig = lane & 3;
      float* dst = part + (size_t)g_w * BT * PS + ug_w * 16 + gid;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int b0 = nt * 8 + 2 * tig;
        dst[(size_t)b0 * PS] = acc[nt][0];
        dst[(size_t)(b0 + 1) * PS] = acc[nt][1];
        dst[(size_t)b0 * PS + 8] = acc[nt][2];
        dst[(size_t)(b0 + 1) * PS + 8] = acc[nt][3];
      }
      __syncthreads();
    }
    // After an expired wait the whole CTA leaves the time loop.  It sends nothing further, so every other CTA of the
    // cluster runs into its own bounded wait and leaves the same way; the byte counts of the barriers stay within the
    // few messages already in flight.
    if (quit) { poisoned = true; break; }
  }
  cp_async_wait<0>();
  if constexpr (RS) { if (T > 0) wait_exchange((T - 1) & 1, T - 1, -1, T & 1); }

  // ---- cotangent of the initial states, bias gradient
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    if (!it_ok[i]) continue;
    float rec[2] = {car[i][0][0], car[i][0][1]};
    if (!p.grad_cut) recurrent_sum(i, (T - 1) & 1, rec);
    store_state2(p.ds0, s0_off[i], f32, rec[0], rec[1]);
#pragma unroll
    for (int s = 1; s < S; ++s) store_state2(p.ds0, s0_off[i] + (size_t)s * B * ND, f32, car[i][s][0], car[i][s][1]);
    const int d = (int)(s0_off[i] % D);
#pragma unroll
    for (int g = 0; g < Gt; ++g) {
      atomicAdd(p.dbias + ((size_t)g * N + n) * D + d, dbacc[i][g][0]);
      atomicAdd(p.dbias + ((size_t)g * N + n) * D + d + 1, dbacc[i][g][1]);
    }
  }
  if (CS > 1) { cluster_arrive(); cluster_wait(); }  // no CTA leaves while a copy from or into it may be in flight
}

}  // namespace FRNN_NS
