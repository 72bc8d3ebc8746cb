// Forward time loop: one persistent launch runs all T steps.
//
// Work split.  A cluster of CS CTAs owns one (head, batch tile of BT rows); CTA `c` of the cluster owns the
// hidden units [c*U, (c+1)*U).  Its slice of the recurrent matrix (Gr*U gate rows x D) lives in registers
// as warp-MMA A fragments for the whole sequence: warp (g, ug) holds gate g of 16 units.  Per step
//   wait     (CS > 1) for the h_{t-1} slices of the other CTAs: an mbarrier counts the bytes their bulk
//            copies deliver into this CTA's shared memory -- no cluster-wide barrier, no memory fence;
//   phase A  every warp multiplies its 16 x D slice with h_{t-1} (BT x D, bf16, shared memory) on the
//            tensor cores and drops the fp32 pre-activations into shared memory;
//   phase B  every thread owns fixed (unit pair, batch row) items: it adds Wx_t (prefetched kStages steps
//            ahead with cp.async) and the bias, runs the cell in fp32 with the non-h states carried in
//            registers and writes the new h (bf16) into this CTA's slice of the h_t buffer;
//   push     one thread per peer CTA starts a bulk async copy (cp.async.bulk, shared::cta -> shared::cluster)
//            of the whole slice into the peer's h_t buffer, completing on the peer's mbarrier;
//   states / activation cache go straight to global memory, off the critical path.
//
// Replaces FLASHRNNCellFusedForward (reference flashrnn/flashrnn/fused/flashrnn_fused_forward.cu:146-659)
// and the per-cell FLASHRNNPointwiseForward functions (fused/{lstm,gru,elman,slstm}_fused_pointwise.cuh).
#pragma once
#include "frnn_common.cuh"

namespace FRNN_NS {

// One cell update in fp32.  pre[g] = (R h)[g];  wx[g], bias[g] as laid out by the reference's gate orders
// (vanilla/lstm.py:19, vanilla/gru.py:16-20, vanilla/elman.py:16-20, vanilla/slstm.py:16-18).
// st[]: previous states in, new states out.  cache[]: values kept for the backward pass.
template <int CELL>
__device__ __forceinline__ void cell_forward(const float* pre, const float* wx, const float* bias, float* st,
                                             float* cache) {
  if constexpr ((CELL & kNoopCell) != 0) {  // chain-floor probe: no gate math, values stay bounded
    using C = Cell<CELL>;
    st[0] = 0.25f * (pre[0] + wx[0] + bias[0]);
#pragma unroll
    for (int k = 0; k < C::GC; ++k) cache[k] = st[0];
  } else if constexpr (CELL == CELL_LSTM) {
    const float ig = fast_sigmoid(pre[0] + wx[0] + bias[0]);
    const float fg = fast_sigmoid(pre[1] + wx[1] + bias[1]);
    const float zv = fast_tanh(pre[2] + wx[2] + bias[2]);
    const float og = fast_sigmoid(pre[3] + wx[3] + bias[3]);
    const float c = fg * st[1] + ig * zv;
    st[0] = og * fast_tanh(c);
    st[1] = c;
    cache[0] = ig; cache[1] = fg; cache[2] = zv; cache[3] = og;
  } else if constexpr (CELL == CELL_GRU) {
    const float gr = pre[0] + bias[0];                       // recurrent-only gate
    const float rg = fast_sigmoid(wx[0] + pre[1] + bias[1]);
    const float zg = fast_sigmoid(wx[1] + pre[2] + bias[2]);
    const float nv = fast_tanh(wx[2] + bias[3] + rg * gr);   // input-only gate n
    st[0] = zg * st[0] + (1.f - zg) * nv;
    cache[0] = gr; cache[1] = rg; cache[2] = zg; cache[3] = nv;
  } else if constexpr (CELL == CELL_ELMAN || CELL == CELL_ELMAN_CLIP) {
    st[0] = fast_tanh(pre[0] + wx[0] + bias[0]);
    if constexpr (CELL == CELL_ELMAN_CLIP) cache[0] = st[0];  // h is clamped afterwards: keep the tanh output
  } else {  // sLSTM; "m' = i~ when n == 0" is applied per element (fused/slstm_fused_pointwise.cuh:53-62)
    const float ir = pre[0] + wx[0] + bias[0];
    const float fr = pre[1] + wx[1] + bias[1];
    const float zv = fast_tanh(pre[2] + wx[2] + bias[2]);
    const float og = fast_sigmoid(pre[3] + wx[3] + bias[3]);
    const float lfm = log_sigmoid(fr) + st[3];
    const float mn = (st[2] == 0.f) ? ir : fmaxf(ir, lfm);
    const float ig = fminf(1.f, __expf(ir - mn));
    const float fg = fminf(1.f, __expf(lfm - mn));
    const float c = fg * st[1] + ig * zv;
    const float n = fmaxf(fg * st[2] + ig, 1.f);
    st[0] = og * __fdividef(c, n);
    st[1] = c; st[2] = n; st[3] = mn;
    cache[0] = ig; cache[1] = fg; cache[2] = zv; cache[3] = og; cache[4] = 1.f - fast_sigmoid(fr);
  }
}

// dynamic shared memory of the forward kernel, in bytes
template <int CELL, int NT>
__host__ __device__ constexpr size_t fwd_smem_bytes(int D, int U, int threads) {
  using C = Cell<CELL>;
  constexpr int BT = NT * 8;
  constexpr int IPT = (BT + 4 * C::Gr - 1) / (4 * C::Gr);
  const int CS = D / U;
  const size_t base = (size_t)2 * CS * BT * (U + 8) * 2 + (size_t)BT * (C::Gr * U + 4) * 4 +
                      (size_t)kStages * C::Gw * IPT * ring_row_len(U, BT, threads) * 4 + 32;
  if (D <= 256) return base;
  // streamed kernels: fragments of R kept in shared memory behind the other buffers (16-byte aligned)
  const size_t b16 = (base + 15) / 16 * 16;
  return b16 + (size_t)stream_ksm(D, kStreamKT, threads, b16) * (threads / 32) * 512;
}

// KT = k-steps (16 columns of R each) a warp keeps in registers.  DYN == false: that is the whole row, D = 16 * KT.
// DYN == true (head dims above 256): D is a run-time value and the k-steps beyond KT are streamed from global memory
// (L2) in every time step -- R no longer fits the registers of one cluster.
template <int CELL, int KT, int NT, bool DYN>
__global__ void __launch_bounds__(LaunchBounds<CELL, KT>::threads, LaunchBounds<CELL, KT>::min_blocks) frnn_fwd_kernel(const __grid_constant__ LoopParams p) {
  using C = Cell<CELL>;
  constexpr int Gr = C::Gr, Gw = C::Gw, Gt = C::Gt, S = C::S, GC = C::GC;
  constexpr int BT = NT * 8;
  const int D = DYN ? p.D : KT * 16;
  const int ktot = DYN ? (p.D >> 4) : KT;  // k-steps per row of R
  constexpr int IPT = (BT + 4 * Gr - 1) / (4 * Gr);  // items (unit pair x batch row) per thread
  constexpr int GCA = GC > 0 ? GC : 1;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x;
  const int U = p.U, CS = p.CS, T = p.T, N = p.N, B = p.B;
  const int US = U + 8;             // row pitch (elements) inside an h slice: 16 B of padding keeps ldmatrix conflict-free
  const int SL = BT * US;           // elements per slice
  const int ushift = 31 - __clz(U >> 4);
  const int PS = Gr * U + 4;        // row pitch of the pre-activation tile; == 4 (mod 16) keeps the stores conflict-free
  const int n = blockIdx.z, bt0 = blockIdx.y * BT;
  const uint32_t crank = (CS > 1) ? cluster_ctarank() : 0u;
  const int unit0 = (int)crank * U;
  const size_t ND = (size_t)N * D;
  const int f32 = p.state_f32;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  elem_t* hbuf = reinterpret_cast<elem_t*>(smem_raw);                   // [2][CS][BT][US]
  float* pre = reinterpret_cast<float*>(smem_raw + (size_t)2 * CS * SL * 2);          // [BT][PS]
  const int RL = ring_row_len(U, BT, nthr);  // threads that own items: the ring has one slot row per such thread
  uint32_t* ring = reinterpret_cast<uint32_t*>(pre + (size_t)BT * PS);                // [kStages][Gw][IPT][RL]
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)kStages * Gw * IPT * RL);  // [2]
  volatile int* gave_up = reinterpret_cast<volatile int*>(full + 2);  // set by a thread whose bounded wait expired

  // ---- this warp's slice of R: gate g_w of units [unit0 + 16*ug_w, +16), all D inputs, as A fragments
  const int nUT = U >> 4;
  const int g_w = warp / nUT, ug_w = warp - g_w * nUT;
  uint4 Rreg[KT];
  const uint4* rsrc = p.Rpack + ((((size_t)n * Gr + g_w) * ktot + (unit0 / 16 + ug_w)) * ktot) * 32 + lane;
#pragma unroll
  for (int k = 0; k < KT; ++k) Rreg[k] = __ldg(rsrc + k * 32);
  // streamed kernels: the next `ksm` k-steps of this warp's fragments stay in shared memory (each lane reads back only
  // what it wrote itself), the rest is re-read from L2 in every step
  int ksm = 0;
  const uint4* rsm = nullptr;
  if constexpr (DYN) {
    const size_t base = (size_t)2 * CS * SL * 2 + (size_t)BT * PS * 4 + (size_t)kStages * Gw * IPT * RL * 4 + 32;
    const size_t b16 = (base + 15) / 16 * 16;  // as fwd_smem_bytes lays it out
    ksm = stream_ksm(D, KT, nthr, b16);
    uint4* mine = reinterpret_cast<uint4*>(smem_raw + b16) + (size_t)warp * ksm * 32 + lane;
    for (int k = 0; k < ksm; ++k) mine[(size_t)k * 32] = __ldg(rsrc + (size_t)(KT + k) * 32);
    rsm = mine - (size_t)KT * 32;  // indexed by the k-step itself, like rsrc
  }

  // ---- this thread's items: everything that does not change over time is computed once
  const int half_u = U >> 1, nitems = half_u * BT;
  const size_t cta_lin = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  bool it_on[IPT], it_ok[IPT];
  const float* pre_it[IPT];            // &pre[bl][2*up]
  uint32_t hloc_it[IPT];               // element offset of (bl, 2*up) inside this CTA's slice
  const elem_t* wx_pf[IPT];     // Wx of the next step to prefetch
  unsigned char* st_ptr[IPT];          // states[0][b][t][n][d] of the current step (bytes)
  uint32_t* ch_ptr[IPT];               // activation cache of the current step
  float bias[IPT][Gt][2], st[IPT][S][2];
  const size_t st_esz = f32 ? 4 : 2;
  const size_t st_sstride = (size_t)B * T * ND * st_esz;        // bytes between states s and s+1
  const size_t ch_step = (size_t)gridDim.x * gridDim.y * gridDim.z * GCA * nitems;  // uint32 per time step
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int q = tid + i * nthr;
    it_on[i] = q < nitems;
    const int bl = it_on[i] ? q / half_u : 0, up = it_on[i] ? q - bl * half_u : 0;
    const int bg = bt0 + bl, d = unit0 + 2 * up;
    it_ok[i] = it_on[i] && bg < B;
    const int bgc = bg < B ? bg : B - 1;
    pre_it[i] = pre + (size_t)bl * PS + 2 * up;
    hloc_it[i] = (uint32_t)(bl * US + 2 * up);
    wx_pf[i] = p.Wx + (size_t)bgc * p.wx_sb + (size_t)n * p.wx_sn + d;
    st_ptr[i] = static_cast<unsigned char*>(p.states) + (((size_t)bgc * T) * ND + (size_t)n * D + d) * st_esz;
    ch_ptr[i] = reinterpret_cast<uint32_t*>(p.cache) + cta_lin * GCA * nitems + (it_on[i] ? q : 0);
#pragma unroll
    for (int g = 0; g < Gt; ++g) {
      const float2 bv = unpack_x2(*reinterpret_cast<const uint32_t*>(p.bias + ((size_t)g * N + n) * D + d));
      bias[i][g][0] = bv.x; bias[i][g][1] = bv.y;
    }
#pragma unroll
    for (int s = 0; s < S; ++s) {
      float2 v = make_float2(0.f, 0.f);
      if (it_ok[i]) v = load_state2(p.s0, ((size_t)s * B + bg) * ND + (size_t)n * D + d, f32);
      st[i][s][0] = v.x; st[i][s][1] = v.y;
    }
  }

  // ---- h_{-1} of the whole head for this batch tile -> hbuf[0] (all slices, read straight from global)
  for (int idx = tid; idx < BT * (D / 2); idx += nthr) {
    const int bl = idx / (D / 2), dp = idx - bl * (D / 2);
    const int bg = bt0 + bl, k = 2 * dp;
    float2 v = make_float2(0.f, 0.f);
    if (bg < B) v = load_state2(p.s0, ((size_t)bg) * ND + (size_t)n * D + k, f32);
    *reinterpret_cast<uint32_t*>(hbuf + (size_t)(k / U) * SL + bl * US + (k % U)) = pack_x2(v.x, v.y);
  }

  // ---- Wx prefetch ring: stage s <- step s
  auto issue_wx = [&](bool live, int stage) {
    if (live) {
#pragma unroll
      for (int i = 0; i < IPT; ++i) {
        if (it_ok[i]) {
#pragma unroll
          for (int g = 0; g < Gw; ++g)
            cp_async4(ring + ((size_t)(stage * Gw + g) * IPT + i) * RL + tid, wx_pf[i] + (size_t)g * p.wx_sg);
          wx_pf[i] += p.wx_st;
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < IPT; ++i)
    if (it_on[i] && !it_ok[i])  // rows beyond B: their inputs read as zero
      for (int s = 0; s < kStages; ++s)
#pragma unroll
        for (int g = 0; g < Gw; ++g) ring[((size_t)(s * Gw + g) * IPT + i) * RL + tid] = 0u;
#pragma unroll
  for (int s = 0; s < kStages; ++s) issue_wx(s < T, s);

  // ---- cluster set-up: mbarriers that count the bytes delivered into hbuf[x]
  const uint32_t slice_bytes = (uint32_t)(SL * 2);
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
    cluster_wait();  // every CTA of the cluster is resident, its barriers initialised and hbuf[0] written
  } else {
    __syncthreads();
  }
  const uint32_t my_slice0 = smem_u32(hbuf + (size_t)crank * SL);   // this CTA's slice in buffer 0
  const uint32_t buf_bytes = (uint32_t)(CS * SL * 2);               // distance to the same slice in buffer 1
  const uint32_t full_u32 = smem_u32(&full[0]);

  for (int t = 0; t < T; ++t) {
    const int cur = t & 1, nxt = cur ^ 1, stage = t % kStages;
    if (CS > 1 && t > 0) {
      if (!mbar_wait_bounded(&full[cur], ((t - 1) >> 1) & 1)) {
        poisoned = true;
        *gave_up = 1;
        report_timeout(p.status, t);
      }
      // re-arm for h_{t+1}; never after an expired wait: that phase is still open and has no arrival left to give
      if (tid == 0 && !poisoned && t + 2 < T) mbar_arrive_expect_tx(&full[cur], expect_bytes);
    }
    // ---------------- phase A: pre[b][g*U + u] = sum_k R[g][u][k] * h_{t-1}[b][k]
    {
      float acc[NT][4];
      warp_mma_rows<KT, NT>(Rreg, hbuf + (size_t)cur * CS * SL, US, 0, ushift, SL, lane, acc);
      if constexpr (DYN) {
        warp_mma_stream<NT, true>(rsm, KT, KT + ksm, hbuf + (size_t)cur * CS * SL, US, 0, ushift, SL, lane, acc);
        warp_mma_stream<NT>(rsrc, KT + ksm, ktot, hbuf + (size_t)cur * CS * SL, US, 0, ushift, SL, lane, acc);
      }
      const int gid = lane >> 2, tig = lane & 3;
      float* dst = pre + g_w * U + ug_w * 16 + gid;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int b0 = nt * 8 + 2 * tig;
        dst[(size_t)b0 * PS] = acc[nt][0];
        dst[(size_t)(b0 + 1) * PS] = acc[nt][1];
        dst[(size_t)b0 * PS + 8] = acc[nt][2];
        dst[(size_t)(b0 + 1) * PS + 8] = acc[nt][3];
      }
    }
    __syncthreads();
    // Set when a wait of this step expired in some thread of the CTA.  The flag was written before the barrier above,
    // so every thread reads the same value; the CTA acts on it at the end of the step, where the load has long landed.
    const int quit = (CS > 1) ? *gave_up : 0;
    // ---------------- phase B: cell update of this thread's items; new h into this CTA's slice of hbuf[nxt]
    cp_async_wait<kStages - 1>();
    float cch[IPT][GCA][2];
    elem_t* hdst = hbuf + (size_t)nxt * CS * SL + (size_t)crank * SL;
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_on[i]) continue;
      float prv[2][Gr], wxv[2][Gw];
#pragma unroll
      for (int g = 0; g < Gr; ++g) {
        const float2 v = *reinterpret_cast<const float2*>(pre_it[i] + g * U);
        prv[0][g] = v.x; prv[1][g] = v.y;
      }
#pragma unroll
      for (int g = 0; g < Gw; ++g) {
        const float2 v = unpack_x2(ring[((size_t)(stage * Gw + g) * IPT + i) * RL + tid]);
        wxv[0][g] = v.x; wxv[1][g] = v.y;
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float sv[S], bv[Gt], cv[GCA];
#pragma unroll
        for (int s = 0; s < S; ++s) sv[s] = st[i][s][e];
#pragma unroll
        for (int g = 0; g < Gt; ++g) bv[g] = bias[i][g][e];
        cell_forward<CELL>(prv[e], wxv[e], bv, sv, cv);
        if (p.fclip > 0.f) sv[0] = clampf(sv[0], p.fclip);
        if (!it_ok[i]) {  // rows beyond B: keep everything zero
#pragma unroll
          for (int s = 0; s < S; ++s) sv[s] = 0.f;
        }
#pragma unroll
        for (int s = 0; s < S; ++s) st[i][s][e] = sv[s];
#pragma unroll
        for (int k = 0; k < GC; ++k) cch[i][k][e] = cv[k];
      }
      const uint32_t hv = pack_x2(st[i][0][0], st[i][0][1]);
      // the recurrence continues from the bf16-rounded h, the value every consumer of `states` sees
      if (!f32) { const float2 r = unpack_x2(hv); st[i][0][0] = r.x; st[i][0][1] = r.y; }
      *reinterpret_cast<uint32_t*>(hdst + hloc_it[i]) = hv;
    }
    if (CS > 1) fence_proxy_async_smem();  // make the slice visible to the bulk-copy engine
    __syncthreads();
    // ---------------- push: this CTA's slice of h_t -> hbuf[nxt] of every other CTA of the cluster
    // (test hook: CTA 0 may withhold its message of step 1 so that the peers' bounded waits can be seen to expire)
    if (CS > 1 && t + 1 < T && !(p.test_drop && crank == 0 && t == 1))  // uniform branch; one elected lane per warp copies
      push_slice_to_peers(my_slice0 + nxt * buf_bytes, slice_bytes, full_u32 + nxt * 8, crank, (uint32_t)CS,
                          (uint32_t)warp, (uint32_t)(nthr >> 5));
    // ---------------- off the critical path: results to global memory, next Wx prefetch
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (!it_ok[i]) continue;
#pragma unroll
      for (int s = 0; s < S; ++s) {
        if (f32) *reinterpret_cast<float2*>(st_ptr[i] + s * st_sstride) = make_float2(st[i][s][0], st[i][s][1]);
        else *reinterpret_cast<uint32_t*>(st_ptr[i] + s * st_sstride) = pack_x2(st[i][s][0], st[i][s][1]);
      }
      st_ptr[i] += ND * st_esz;
      if (GC > 0 && p.cache != nullptr) {
#pragma unroll
        for (int k = 0; k < GC; ++k) ch_ptr[i][(size_t)k * nitems] = pack_x2(cch[i][k][0], cch[i][k][1]);
        ch_ptr[i] += ch_step;
      }
    }
    issue_wx(t + kStages < T, stage);
    // After an expired wait the whole CTA leaves the time loop.  It sends nothing further, so every other CTA of the
    // cluster runs into its own bounded wait and leaves the same way; the byte counts of the barriers stay within the
    // few messages already in flight.
    if (quit) break;
  }
  cp_async_wait<0>();
  if (CS > 1) { cluster_arrive(); cluster_wait(); }  // no CTA leaves while a copy from or into it may be in flight
}

}  // namespace FRNN_NS
