// Time loops for LARGE batches on the 5th-generation tensor cores: one CTA owns a whole head (head dim 64) and a tile
// of 128 batch rows for all T steps.  Elman cell (h_t = tanh(Wx_t + R h_{t-1} + b)).
//
// Forward, per step:  acc[128 x 64] (fp32, tensor memory) = Wx_t * I + 1 * b  (issued ahead, off the critical path)
//                     acc += h_{t-1} * R^T                                     (tcgen05.mma, operands in shared memory)
//                     h_t = tanh(acc) -> bf16 tile in shared memory            (tcgen05.ld, one batch row per thread)
//   The h tile is the A operand of the next step and the source of a tensor-map bulk store into `states`; Wx tiles are
//   fetched by tensor-map bulk loads a few steps ahead.  Identity and bias products put the additions on the tensor pipe,
//   so the 128 row threads only do tanh, the bf16 packing and eight 16-byte shared-memory stores per step.
// Backward, per step: acc = dh_ext_t * I (ahead) + delta_{t+1} * R;  delta_t = acc * (1 - h_t^2) -> bf16 tile;
//                     dR (tensor memory, kept for all T steps) += delta_t^T * h_{t-1};  delta tile -> dWx (bulk store);
//                     db in registers.  No separate dR pass over HBM: the delta and h tiles are in shared memory anyway.
// Warps 0-3: one batch row per thread.  Warp 4, one lane: issues every bulk copy and every MMA.  All tiles are
// [128 rows][64 bf16] = rows of 128 bytes in the 128-byte-swizzle layout shared by the bulk copies and the MMA descriptors.
// When the batch is a multiple of 8 (and T >= 2) every bulk copy moves TWO time steps: batch rows lie T*N*128 bytes apart
// (one 2 MB page each at the sizes this path is for), address translation bounds the copies, and the second touch of a
// page right after the first one is cheap.  The tiles of the two steps then interleave in shared memory by 8-row group.
//
// Replaces, for these shapes, FLASHRNNCellFusedForward / FLASHRNNCellFusedBackward and the dR GEMM + bias reduction that
// follow the reverse loop (flashrnn/flashrnn/fused/flashrnn_fused_forward.cu:146-659, flashrnn_fused_backward.cu:129-624,
// 626-665, 1049-1058; cell: fused/elman_fused_pointwise.cuh:34-93).
#include "frnn_aux.cuh"
#include "frnn_tc.cuh"
#include "frnn_tmap.cuh"

namespace FRNN_NS {

namespace {

constexpr int WD = 64;                          // head dim
constexpr int WM = 128;                         // batch rows per CTA = UMMA M
constexpr uint32_t WTILE = WM * WD * 2;         // bytes of a [128][64] bf16 tile
constexpr uint32_t WMAT = WD * WD * 2;          // bytes of a [64][64] bf16 operand
constexpr int WF_STAGES = 8;                    // forward: Wx tiles in flight
constexpr int WB_STAGES = 4;                    // backward: h tiles and cotangent tiles in flight (each)
constexpr int W_THREADS = 160;

// byte offset of 16-byte chunk `chunk` of row `row` inside a 128-byte-swizzled tile
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

// the same inside a two-step buffer, where the 8-row groups of the two tiles interleave (group g of the tile in slot s at
// g * 2048 + s * 1024): how a tensor-map box of [16 groups][2 steps][8 rows][128 bytes] lands in shared memory
__device__ __forceinline__ uint32_t sw128_pair(uint32_t row, uint32_t chunk, uint32_t slot) {
  return (row >> 3) * 2048u + slot * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(pack_x2(v[0], v[1]), pack_x2(v[2], v[3]), pack_x2(v[4], v[5]), pack_x2(v[6], v[7]));
}

// ================================================================================================ forward
struct WideFwdParams {
  const elem_t* R;     // [1,N,64,64]
  const elem_t* bias;  // [1,N,64]
  const elem_t* s0;    // [1,B,1,N,64]
  unsigned* status;
  int B, T, N;
  int test_drop;  // test hook: the copy of one tile (step index 2) is announced to its barrier but never issued
};

constexpr uint32_t WF_OFF_WX = 0;
constexpr uint32_t WF_OFF_H = WF_OFF_WX + WF_STAGES * WTILE;
constexpr uint32_t WF_OFF_R = WF_OFF_H + 4 * WTILE;  // h tiles: h_t lives in tile t % 3, or in slot t & 1 of one of two two-step buffers
constexpr uint32_t WF_OFF_I = WF_OFF_R + WMAT;
constexpr uint32_t WF_OFF_ONES = WF_OFF_I + WMAT;       // A operand [128 rows][16 k], k = 0 holds 1.0 (no swizzle)
constexpr uint32_t WF_OFF_BIAS = WF_OFF_ONES + 4096;    // B operand [64 rows][16 k], k = 0 holds b[row] (no swizzle)
constexpr uint32_t WF_OFF_BAR = WF_OFF_BIAS + 2048;
constexpr uint32_t WF_SMEM = WF_OFF_BAR + 8 * (WF_STAGES + 3) + 16 + 1024;  // + slack for the 1024-byte alignment

// PAIR: every bulk copy moves two time steps of 8-row groups (maps of map_pairs): each batch row is its own 2 MB page
// (rows lie T*N*128 bytes apart), and touching a page twice in a row halves the address translations that miss.
template <bool PAIR>
__global__ void __launch_bounds__(W_THREADS, 1)
wide_fwd_elman_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_states,
                      const WideFwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_raw + (base - raw);
  uint64_t* wx_full = reinterpret_cast<uint64_t*>(sm + WF_OFF_BAR);  // [WF_STAGES] bytes of a Wx tile have landed
  uint64_t* acc_full = wx_full + WF_STAGES;                          // [2] MMAs into accumulator x have completed
  uint64_t* h_ready = acc_full + 2;                                  // 128 arrivals: h_t is in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(h_ready + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.y, b0 = blockIdx.x * WM, T = p.T;

  // ---- operands written once: R (as [d][p], K-major), the identity, the ones column, the bias row, h_{-1}
  {
    const elem_t* Rn = p.R + (size_t)n * WD * WD;
    for (int c = tid; c < WD * 8; c += W_THREADS) {
      const uint32_t d = c >> 3, j = c & 7;
      *reinterpret_cast<uint4*>(sm + WF_OFF_R + sw128(d, j)) = *reinterpret_cast<const uint4*>(Rn + d * WD + j * 8);
      const uint32_t w = (d & 7) >> 1, one = ((d >> 3) == j) ? (kOneBits << (16 * (d & 1))) : 0u;  // 1.0 at k = d
      *reinterpret_cast<uint4*>(sm + WF_OFF_I + sw128(d, j)) =
          make_uint4(w == 0 ? one : 0u, w == 1 ? one : 0u, w == 2 ? one : 0u, w == 3 ? one : 0u);
    }
    for (int r = tid; r < WM; r += W_THREADS) {
      unsigned char* q = sm + WF_OFF_ONES + (r >> 3) * 256 + (r & 7) * 16;
      *reinterpret_cast<uint4*>(q) = make_uint4(kOneBits, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(q + 128) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int d = tid; d < WD; d += W_THREADS) {
      unsigned char* q = sm + WF_OFF_BIAS + (d >> 3) * 256 + (d & 7) * 16;
      *reinterpret_cast<uint4*>(q) = make_uint4(elem_bits(p.bias[(size_t)n * WD + d]), 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(q + 128) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (tid < WM) {  // h_{-1} -> h tile 2 (step t reads tile (t + 2) % 3 and writes tile t % 3); PAIR: slot 1 of buffer 0
      const int b = b0 + tid;
      const uint4* src = reinterpret_cast<const uint4*>(p.s0 + ((size_t)(b < p.B ? b : 0) * p.N + n) * WD);
#pragma unroll
      for (uint32_t j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(sm + WF_OFF_H + (PAIR ? sw128_pair(tid, j, 1) : 2 * WTILE + sw128(tid, j))) =
            (b < p.B) ? src[j] : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (tid == 0) {
    for (int s = 0; s < WF_STAGES; ++s) mbar_init(&wx_full[s], 1);
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_full[1], 1);
    mbar_init(h_ready, WM);
    fence_mbar_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, 128);  // two accumulators of 64 fp32 columns
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer: bulk copies and MMAs
      const uint32_t idesc = instr_desc_16(WM, WD, 0, 0);
      const void* tmw = &tm_wx;
      const void* tms = &tm_states;
      // descriptor halves: the low word carries the address (16-byte units), the high word is a constant of the layout
      constexpr uint32_t HI = desc_hi(1024, true), HIP = desc_hi(256, false), TILE16 = WTILE >> 4;
      const uint32_t wx_lo = (base + WF_OFF_WX) >> 4, h_lo = (base + WF_OFF_H) >> 4, r_lo = (base + WF_OFF_R) >> 4,
                     i_lo = (base + WF_OFF_I) >> 4, ones_lo = ((base + WF_OFF_ONES) >> 4) | ((128u >> 4) << 16),
                     bias_lo = ((base + WF_OFF_BIAS) >> 4) | ((128u >> 4) << 16);
      if constexpr (PAIR) {
        // h_t: buffer ((t + 2) >> 1) & 1, slot t & 1;  Wx_t: buffer (t >> 1) % NP, slot t & 1
        constexpr uint32_t HI2 = desc_hi(2048, true), PAIR16 = (2 * WTILE) >> 4, SLOT16 = 1024 >> 4;
        constexpr int NP = WF_STAGES / 2;
        const int P = (T + 1) >> 1, bh = b0 >> 3;
        int loads = 0, seen = 0;  // two-step boxes of Wx requested / seen to land
        auto load_pair = [&](int q) {
          const int s = q % NP;
          mbar_arrive_expect_tx(&wx_full[s], 2 * WTILE);
          if (!(p.test_drop && q == 1)) tma_load_5d(base + WF_OFF_WX + s * 2 * WTILE, tmw, 0, 0, 2 * q, bh, n, &wx_full[s]);
          ++loads;
        };
        auto wait_pair = [&](int q) {
          if (!mbar_wait_bounded(&wx_full[q % NP], (uint32_t)((q / NP) & 1))) return false;
          seen = q + 1;
          return true;
        };
        auto issue_pre = [&](int t) {  // acc[t & 1] = Wx_t * I + ones * bias
          const uint32_t a = wx_lo + ((t >> 1) % NP) * PAIR16 + (t & 1) * SLOT16, d = tmem + (t & 1) * WD;
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI2, i_lo + 2 * k, HI, idesc, k);
          umma_parts(d, ones_lo, HIP, bias_lo, HIP, idesc, 1u);
        };
        for (int q = 0; q < P && q < NP; ++q) load_pair(q);
        bool ok = wait_pair(0);
        if (ok) issue_pre(0);
        else report_timeout(p.status, 0);
        for (int t = 0; ok && t < T; ++t) {
          if (t > 0) {
            if (!mbar_wait_bounded(h_ready, (uint32_t)((t - 1) & 1))) { report_timeout(p.status, t); ok = false; break; }
            tc_fence_after();
          }
          // steps t and t+1 (t even) overwrite the buffer of h_{t-4}, h_{t-3}, whose store was issued two steps ago
          if (!(t & 1)) bulk_wait_group_read<0>();
          const uint32_t hb = (uint32_t)((t + 1) >> 1) & 1u;  // buffer of h_{t-1}
          const uint32_t a = h_lo + hb * PAIR16 + ((t - 1) & 1) * SLOT16, d = tmem + (t & 1) * WD;
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI2, r_lo + 2 * k, HI, idesc, 1u);
          umma_commit(&acc_full[t & 1]);
          if (t > 0 && !(t & 1)) {
            // h_{t-2}, h_{t-1} -> states[0][b0.., t-2 .. t-1, n, :]; the Wx box of those steps was consumed by MMAs that
            // completed before h_{t-1} could be computed
            tma_store_5d(tms, base + WF_OFF_H + hb * 2 * WTILE, 0, 0, t - 2, bh, n);
            bulk_commit_group();
            const int q = (t >> 1) - 1 + NP;
            if (q < P) load_pair(q);
          }
          if (t + 1 < T) {
            if (!((t + 1) & 1) && !wait_pair((t + 1) >> 1)) { report_timeout(p.status, t); ok = false; break; }
            issue_pre(t + 1);
          }
        }
        if (ok) {
          if (mbar_wait_bounded(h_ready, (uint32_t)((T - 1) & 1))) {
            // the last box: steps T-2, T-1, or step T-1 alone (T odd; the store clips the second tile)
            tma_store_5d(tms, base + WF_OFF_H + ((uint32_t)((T + 1) >> 1) & 1u) * 2 * WTILE, 0, 0, (T - 1) & ~1, bh, n);
            bulk_commit_group();
          } else {
            report_timeout(p.status, T);
          }
        }
        for (int i = (seen > loads - NP ? seen : loads - NP); i < loads; ++i)
          mbar_wait_bounded(&wx_full[i % NP], (uint32_t)((i / NP) & 1));
        bulk_wait_group<0>();
      } else {
      int loads = 0, waited = 0;  // Wx tiles requested / seen to land (both in step order)
      int ls = 0;                 // ring slot of the next request
      int cs = 0;                 // ring slot and barrier parity of the next tile to consume
      uint32_t cpar = 0;
      auto load_wx = [&](int t) {
        mbar_arrive_expect_tx(&wx_full[ls], WTILE);
        if (!(p.test_drop && t == 2)) tma_load_5d(base + WF_OFF_WX + ls * WTILE, tmw, 0, n, 0, t, b0, &wx_full[ls]);
        ls = (ls + 1 == WF_STAGES) ? 0 : ls + 1;
        ++loads;
      };
      auto wait_wx = [&]() { return mbar_wait_bounded(&wx_full[cs], cpar); };
      auto issue_pre = [&](int t) {  // acc[t & 1] = Wx_t * I + ones * bias, from ring slot cs
        const uint32_t a = wx_lo + cs * TILE16, d = tmem + (t & 1) * WD;
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI, i_lo + 2 * k, HI, idesc, k);
        umma_parts(d, ones_lo, HIP, bias_lo, HIP, idesc, 1u);
        ++waited;
        if (++cs == WF_STAGES) { cs = 0; cpar ^= 1u; }
      };
      for (int t = 0; t < T && t < WF_STAGES; ++t) load_wx(t);
      bool ok = wait_wx();
      if (ok) issue_pre(0);
      else report_timeout(p.status, 0);
      int hr = 2;  // tile holding h_{t-1}
      for (int t = 0; ok && t < T; ++t) {
        if (t > 0) {
          if (!mbar_wait_bounded(h_ready, (uint32_t)((t - 1) & 1))) { report_timeout(p.status, t); ok = false; break; }
          tc_fence_after();
        }
        // step t's threads overwrite the tile of h_{t-3}: its store (two groups back) must have left shared memory; with
        // three tiles the store gets two whole steps for that, and this wait is off the critical path
        bulk_wait_group_read<1>();
        const uint32_t a = h_lo + hr * TILE16, d = tmem + (t & 1) * WD;
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI, r_lo + 2 * k, HI, idesc, 1u);
        umma_commit(&acc_full[t & 1]);
        if (t > 0) {  // h_{t-1} -> states[0][b0.., t-1, n, :]
          tma_store_5d(tms, base + WF_OFF_H + hr * WTILE, 0, n, t - 1, b0, 0);
          bulk_commit_group();
          // the Wx tile of step t-1 was consumed by MMAs that completed before h_{t-1} could be computed
          if (t - 1 + WF_STAGES < T) load_wx(t - 1 + WF_STAGES);
        }
        if (t + 1 < T) {
          if (!wait_wx()) {
            report_timeout(p.status, t);
            ok = false;
            break;
          }
          issue_pre(t + 1);
        }
        hr = (hr == 2) ? 0 : hr + 1;
      }
      if (ok) {
        if (mbar_wait_bounded(h_ready, (uint32_t)((T - 1) & 1))) {
          tma_store_5d(tms, base + WF_OFF_H + hr * WTILE, 0, n, T - 1, b0, 0);
          bulk_commit_group();
        } else {
          report_timeout(p.status, T);
        }
      }
      // never leave with copies in flight (only an expired wait leaves any load unobserved)
      for (int i = (waited > loads - WF_STAGES ? waited : loads - WF_STAGES); i < loads; ++i)
        mbar_wait_bounded(&wx_full[i % WF_STAGES], (uint32_t)((i / WF_STAGES) & 1));
      bulk_wait_group<0>();
      }
    }
  } else {
    // ------------------------------------------------------------ row threads: h_t = tanh(acc)
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    int hw = 0;  // tile that receives h_t
    for (int t = 0; t < T; ++t) {
      if (!mbar_wait_bounded(&acc_full[t & 1], (uint32_t)((t >> 1) & 1))) { report_timeout(p.status, t); break; }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld64(trow + (t & 1) * WD, r0, r1);
      unsigned char* dst = sm + WF_OFF_H + (PAIR ? (uint32_t)((t + 2) >> 1 & 1) * 2 * WTILE : hw * WTILE);
      hw = (hw == 2) ? 0 : hw + 1;
#pragma unroll
      for (uint32_t j = 0; j < 8; ++j) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = fast_tanh(__uint_as_float(j < 4 ? r0[j * 8 + i] : r1[(j - 4) * 8 + i]));
        *reinterpret_cast<uint4*>(dst + (PAIR ? sw128_pair(tid, j, t & 1) : sw128(tid, j))) = pack8(v);
      }
      fence_proxy_async_smem();  // the tile is read by the tensor core and by the bulk store
      tc_fence_before();
      mbar_arrive(h_ready);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, 128);
  }
}


// ================================================================================================ LSTM / GRU forward
// The same loop for the multi-gate cells at head dim 64, described for the four-gate LSTM cell (the GRU differs as noted
// at the kernel): the accumulator of a step is [128 rows][4 gates x 64] fp32 = 256 columns of tensor memory (two of
// them alternate), filled by
//   acc      = 1 * b  (one MMA, N = 256, overwriting);  acc[:, g] += Wx_t[g] * I  (4 gates x 4 MMAs, N = 64)  -- issued ahead
//   acc     += h_{t-1} * R^T                            (4 MMAs, N = 256; R as [4*64 rows][64 k])
// Two row threads per batch row (8 warps, two per scheduler; a warp reads the tensor-memory lanes of its quarter, so
// warps w and w + 4 share 32 rows and split the 64 units) read the accumulator 16 units at a time (4 gates x 16 columns),
// keep the cell state c of their 32 units in registers (fp32) and write h_t into the shared-memory tile that the next
// step multiplies and a bulk store sends to `states[0]`.  After the arrival that hands h_t on, c_t and the four cached
// activations go straight to global memory: a thread owns 64 contiguous bytes per value kind, neighbouring lanes swap
// halves, and each 32-byte store instruction covers 16 rows x 64 bytes.  The activation cache is written in the layout of
// the REVERSE loop's own tile (one CTA per head, 16 batch rows: frnn_bwd_kernel reads it as it reads its forward
// kernel's), so only the forward loop changes.
// Wx_t arrives as one tensor-map copy of [4 gates][128 rows][64] per step into a ring of two 64 KB stages; the stage of
// step t is refilled with step t+2 as soon as the step's MMAs are known to have completed.
struct WideGatesParams {
  const elem_t* R;     // [4,N,64,64]
  const elem_t* bias;  // [4,N,64]
  const elem_t* s0;    // [2,B,1,N,64]
  elem_t* states;      // [2,B,T,N,64]; h leaves through the tensor map, c through plain stores
  uint32_t* cache;     // reverse loop's layout (16-row tiles): [t][head][tile][slot][row in tile][unit pair]; or null
  unsigned* status;
  int B, T, N;
  int test_drop;  // test hook: the copy of one Wx box (step index 2) is announced to its barrier but never issued
  float fclip;    // > 0: the new h is clamped to [-fclip, fclip]
};
constexpr int WL_G = 4;
constexpr int WL_THREADS = 288;  // warps 0-7: two row threads per batch row; warp 8, one lane: every bulk copy and MMA
constexpr uint32_t WL_OFF_WX = 0;                                   // 2 stages x 4 gate tiles
constexpr uint32_t WL_OFF_H = WL_OFF_WX + 2 * WL_G * WTILE;         // h_t in tile t & 1
constexpr uint32_t WL_OFF_R = WL_OFF_H + 2 * WTILE;                 // [256][64] K-major, 128-byte swizzle
constexpr uint32_t WL_OFF_I = WL_OFF_R + WL_G * WMAT;
constexpr uint32_t WL_OFF_ONES = WL_OFF_I + WMAT;                   // A operand [128 rows][16 k], k = 0 holds 1.0
constexpr uint32_t WL_OFF_BIAS = WL_OFF_ONES + 4096;                // B operand [256 rows][16 k], k = 0 holds b[row]
constexpr uint32_t WL_OFF_BAR = WL_OFF_BIAS + 8192;
constexpr uint32_t WL_SMEM = WL_OFF_BAR + 8 * 8 + 16 + 1024;
static_assert(WL_SMEM <= 227 * 1024, "shared memory of the LSTM loop");

// one 256-bit store (32-byte aligned address)
__device__ __forceinline__ void st_global_32B(void* q, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(q), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x),
               "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}

// 4 x 16 consecutive fp32 columns (the four gates of 16 units), one wait
__device__ __forceinline__ void tmem_ld16x4(uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3, uint32_t (&a)[16], uint32_t (&b)[16],
                                            uint32_t (&c)[16], uint32_t (&d)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%65];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47}, [%66];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%67];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]),
        "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]), "=r"(c[4]), "=r"(c[5]), "=r"(c[6]), "=r"(c[7]), "=r"(c[8]), "=r"(c[9]), "=r"(c[10]), "=r"(c[11]), "=r"(c[12]), "=r"(c[13]), "=r"(c[14]), "=r"(c[15]),
        "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
      : "r"(t0), "r"(t1), "r"(t2), "r"(t3) : "memory");
}

// CELL: CELL_LSTM, or CELL_GRU -- three input gates (r, z, n) and three recurrent ones (g~, r, z): accumulator columns
// [g~ | r | z | n] = [R0 h + b0 | Wx0 + R1 h + b1 | Wx1 + R2 h + b2 | Wx2 + b3], so the recurrent product covers the first
// 192 columns, the input gates the last 192, and the row threads carry h instead of c.
template <int CELL>
__global__ void __launch_bounds__(WL_THREADS, 1)
wide_fwd_gates_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_states, const WideGatesParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_raw + (base - raw);
  uint64_t* wx_full = reinterpret_cast<uint64_t*>(sm + WL_OFF_BAR);  // [2] bytes of a Wx stage have landed
  uint64_t* acc_full = wx_full + 2;                                  // [2] MMAs into accumulator x have completed
  uint64_t* h_ready = acc_full + 2;                                  // 256 arrivals: h_t is in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(h_ready + 1);

  constexpr bool GRU = CELL == CELL_GRU;
  constexpr int NGW = GRU ? 3 : 4;         // gates of Wx
  constexpr int NGR = GRU ? 3 : 4;         // gates of R
  constexpr uint32_t WX_COL0 = GRU ? WD : 0;  // accumulator column of the first Wx gate
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.y, b0 = blockIdx.x * WM, T = p.T, N = p.N, B = p.B;

  // ---- operands written once
  for (int c = tid; c < NGR * WD * 8; c += WL_THREADS) {  // R: row j = g * 64 + d holds R[g][n][d][:]
    const uint32_t j = c >> 3, q = c & 7, g = j >> 6, d = j & 63;
    *reinterpret_cast<uint4*>(sm + WL_OFF_R + sw128(j, q)) =
        *reinterpret_cast<const uint4*>(p.R + (((size_t)g * N + n) * WD + d) * WD + q * 8);
  }
  for (int c = tid; c < WD * 8; c += WL_THREADS) {  // identity: 1.0 at k = d
    const uint32_t d = c >> 3, j = c & 7;
    const uint32_t w = (d & 7) >> 1, one = ((d >> 3) == j) ? (kOneBits << (16 * (d & 1))) : 0u;
    *reinterpret_cast<uint4*>(sm + WL_OFF_I + sw128(d, j)) =
        make_uint4(w == 0 ? one : 0u, w == 1 ? one : 0u, w == 2 ? one : 0u, w == 3 ? one : 0u);
  }
  for (int r = tid; r < WM; r += WL_THREADS) {
    unsigned char* q = sm + WL_OFF_ONES + (r >> 3) * 256 + (r & 7) * 16;
    *reinterpret_cast<uint4*>(q) = make_uint4(kOneBits, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(q + 128) = make_uint4(0u, 0u, 0u, 0u);
  }
  for (int j = tid; j < WL_G * WD; j += WL_THREADS) {
    unsigned char* q = sm + WL_OFF_BIAS + (j >> 3) * 256 + (j & 7) * 16;
    *reinterpret_cast<uint4*>(q) = make_uint4(elem_bits(p.bias[((size_t)(j >> 6) * N + n) * WD + (j & 63)]), 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(q + 128) = make_uint4(0u, 0u, 0u, 0u);
  }
  const int row = tid & (WM - 1), half = tid >> 7;  // row threads: two per batch row, units 32 * half .. 32 * half + 31
  const bool row_ok = tid < 2 * WM && b0 + row < B;
  if (tid < WM) {  // h_{-1} -> tile 1 (step t reads tile (t + 1) & 1 and writes tile t & 1)
    const uint4* src = reinterpret_cast<const uint4*>(p.s0 + ((size_t)(row_ok ? b0 + row : 0) * N + n) * WD);
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j)
      *reinterpret_cast<uint4*>(sm + WL_OFF_H + WTILE + sw128(tid, j)) = row_ok ? src[j] : make_uint4(0u, 0u, 0u, 0u);
  }
  if (tid == 0) {
    mbar_init(&wx_full[0], 1);
    mbar_init(&wx_full[1], 1);
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_full[1], 1);
    mbar_init(h_ready, 2 * WM);
    fence_mbar_init();
  }
  if (warp == 8) tmem_alloc(tmem_slot, 512);  // two accumulators of 4 x 64 fp32 columns
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer: bulk copies and MMAs
      const uint32_t idesc64 = instr_desc_16(WM, WD, 0, 0), idesc256 = instr_desc_16(WM, WL_G * WD, 0, 0),
                     idesc_r = instr_desc_16(WM, NGR * WD, 0, 0);
      const void* tmw = &tm_wx;
      const void* tms = &tm_states;
      constexpr uint32_t HI = desc_hi(1024, true), HIP = desc_hi(256, false), TILE16 = WTILE >> 4;
      const uint32_t wx_lo = (base + WL_OFF_WX) >> 4, h_lo = (base + WL_OFF_H) >> 4, r_lo = (base + WL_OFF_R) >> 4,
                     i_lo = (base + WL_OFF_I) >> 4, ones_lo = ((base + WL_OFF_ONES) >> 4) | ((128u >> 4) << 16),
                     bias_lo = ((base + WL_OFF_BIAS) >> 4) | ((128u >> 4) << 16);
      int loads = 0, seen = 0;  // Wx stages requested / seen to land (both in step order)
      auto load_wx = [&](int t) {  // [4 gates][128 rows][64] of step t -> stage t & 1
        mbar_arrive_expect_tx(&wx_full[t & 1], NGW * WTILE);
        if (!(p.test_drop && t == 2))
          tma_load_5d(base + WL_OFF_WX + (uint32_t)(t & 1) * WL_G * WTILE, tmw, 0, b0, 0, n, t, &wx_full[t & 1]);
        ++loads;
      };
      auto wait_wx = [&](int t) {
        if (!mbar_wait_bounded(&wx_full[t & 1], (uint32_t)((t >> 1) & 1))) return false;
        seen = t + 1;
        return true;
      };
      auto issue_pre = [&](int t) {  // acc[t & 1] = ones * bias (all 256 columns, overwriting), then += Wx_t[g] * I per gate
        const uint32_t d = tmem + (uint32_t)(t & 1) * (WL_G * WD), a = wx_lo + (uint32_t)(t & 1) * WL_G * TILE16;
        umma_parts(d, ones_lo, HIP, bias_lo, HIP, idesc256, 0u);
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)NGW; ++g)
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) umma_parts(d + WX_COL0 + g * WD, a + g * TILE16 + 2 * k, HI, i_lo + 2 * k, HI, idesc64, 1u);
      };
      load_wx(0);
      if (T > 1) load_wx(1);
      bool ok = wait_wx(0);
      if (ok) issue_pre(0);
      else report_timeout(p.status, 0);
      for (int t = 0; ok && t < T; ++t) {
        if (t > 0) {
          if (!mbar_wait_bounded(h_ready, (uint32_t)((t - 1) & 1))) { report_timeout(p.status, t); ok = false; break; }
          tc_fence_after();
        }
        // the row threads of step t overwrite the tile of h_{t-2}, whose store was issued a whole step ago
        bulk_wait_group_read<0>();
        const uint32_t a = h_lo + (uint32_t)((t + 1) & 1) * TILE16, d = tmem + (uint32_t)(t & 1) * (WL_G * WD);
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI, r_lo + 2 * k, HI, idesc_r, 1u);
        umma_commit(&acc_full[t & 1]);
        if (t > 0) {  // h_{t-1} -> states[0][b0.., t-1, n, :]
          tma_store_5d(tms, base + WL_OFF_H + (uint32_t)((t - 1) & 1) * WTILE, 0, n, t - 1, b0, 0);
          bulk_commit_group();
        }
        if (t + 1 < T) {
          if (!wait_wx(t + 1)) { report_timeout(p.status, t); ok = false; break; }
          issue_pre(t + 1);
        }
        if (t + 2 < T) {  // the stage of step t is free once its MMAs (all issued before the commit above) have completed
          if (!mbar_wait_bounded(&acc_full[t & 1], (uint32_t)((t >> 1) & 1))) { report_timeout(p.status, t); ok = false; break; }
          load_wx(t + 2);
        }
      }
      if (ok) {
        if (mbar_wait_bounded(h_ready, (uint32_t)((T - 1) & 1))) {
          tma_store_5d(tms, base + WL_OFF_H + (uint32_t)((T - 1) & 1) * WTILE, 0, n, T - 1, b0, 0);
          bulk_commit_group();
        } else {
          report_timeout(p.status, T);
        }
      }
      // never leave with copies in flight (only an expired wait leaves a load unobserved)
      for (int i = (seen > loads - 2 ? seen : loads - 2); i < loads; ++i) mbar_wait_bounded(&wx_full[i & 1], (uint32_t)((i >> 1) & 1));
      bulk_wait_group<0>();
    }
  } else {
    // ------------------------------------------------------------ row threads: half a batch row (32 units) each; a warp
    // reads the tensor-memory lanes of its quarter (warp & 3), so warps w and w + 4 share 32 rows
    const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int b = b0 + row;
    const size_t ND = (size_t)N * WD;
    float cst[32];  // LSTM: cell state c of this half row (fp32 over all steps); GRU: h_{t-1}, as rounded to 16 bits
    {
      const uint4* src = reinterpret_cast<const uint4*>(p.s0 + ((size_t)(GRU ? 0 : B) + (row_ok ? b : 0)) * ND + (size_t)n * WD + 32 * half);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 w = row_ok ? src[j] : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 v = unpack_x2(ww[e]);
          cst[j * 8 + 2 * e] = v.x;
          cst[j * 8 + 2 * e + 1] = v.y;
        }
      }
    }
    // c_t -> states[1][b][t][n][:];  cache: 16-row tiles of the reverse loop, see WideGatesParams.  Pointers to this lane's
    // 32-byte slot (units 32 half + 16 odd ..) in the even and in the odd row of its lane pair.
    const bool odd = (lane & 1) != 0;
    const int be = b & ~1;
    const bool ok_e = be < B, ok_o = be + 1 < B;
    elem_t* c_e = p.states + (((size_t)B + (ok_e ? be : 0)) * T) * ND + (size_t)n * WD + 32 * half + (odd ? 16 : 0);
    elem_t* c_o = c_e + (size_t)T * ND;
    const size_t tiles16 = (size_t)((B + 15) / 16);
    uint32_t* ch_e = p.cache ? p.cache + (((size_t)n * tiles16 + (size_t)(be >> 4)) * WL_G) * 512 + (size_t)(be & 15) * 32 + 16 * half + (odd ? 8 : 0)
                             : nullptr;
    uint32_t* ch_o = ch_e ? ch_e + 32 : nullptr;
    const size_t ch_step = (size_t)N * tiles16 * WL_G * 512;
    for (int t = 0; t < T; ++t) {
      if (!mbar_wait_bounded(&acc_full[t & 1], (uint32_t)((t >> 1) & 1))) { report_timeout(p.status, t); break; }
      tc_fence_after();
      unsigned char* hdst = sm + WL_OFF_H + (uint32_t)(t & 1) * WTILE;
      const uint32_t acc = trow + (uint32_t)(t & 1) * (WL_G * WD);
      uint4 out[1 + WL_G][4];  // c_t and the four activations of this thread's 32 units, packed for the stores below
#pragma unroll
      for (int qq = 0; qq < 2; ++qq) {  // units 16 q .. 16 q + 15
        const int q = 2 * half + qq;
        uint32_t ri[16], rf[16], rz[16], ro[16];
        tmem_ld16x4(acc + 16 * q, acc + WD + 16 * q, acc + 2 * WD + 16 * q, acc + 3 * WD + 16 * q, ri, rf, rz, ro);
        float hv[16], gi[16], gf[16], gz[16], go[16];  // h_t and the four cached values (LSTM: i, f, z, o; GRU: g~, r, z, n)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if constexpr (GRU) {
            gi[j] = __uint_as_float(ri[j]);
            gf[j] = fast_sigmoid(__uint_as_float(rf[j]));
            gz[j] = fast_sigmoid(__uint_as_float(rz[j]));
            go[j] = fast_tanh(__uint_as_float(ro[j]) + gf[j] * gi[j]);
            hv[j] = gz[j] * cst[16 * qq + j] + (1.f - gz[j]) * go[j];
          } else {
            gi[j] = fast_sigmoid(__uint_as_float(ri[j]));
            gf[j] = fast_sigmoid(__uint_as_float(rf[j]));
            gz[j] = fast_tanh(__uint_as_float(rz[j]));
            go[j] = fast_sigmoid(__uint_as_float(ro[j]));
            const float c = gf[j] * cst[16 * qq + j] + gi[j] * gz[j];
            cst[16 * qq + j] = c;
            hv[j] = go[j] * fast_tanh(c);
          }
        }
        if (p.fclip > 0.f) {
#pragma unroll
          for (int j = 0; j < 16; ++j) hv[j] = clampf(hv[j], p.fclip);
        }
        auto pack16 = [](const float (&v)[16], uint4& lo, uint4& hi) {
          lo = make_uint4(pack_x2(v[0], v[1]), pack_x2(v[2], v[3]), pack_x2(v[4], v[5]), pack_x2(v[6], v[7]));
          hi = make_uint4(pack_x2(v[8], v[9]), pack_x2(v[10], v[11]), pack_x2(v[12], v[13]), pack_x2(v[14], v[15]));
        };
        uint4 lo, hi;
        pack16(hv, lo, hi);
        *reinterpret_cast<uint4*>(hdst + sw128(row, 2 * q)) = lo;
        *reinterpret_cast<uint4*>(hdst + sw128(row, 2 * q + 1)) = hi;
        if constexpr (GRU) {  // the recurrence continues from the rounded h, the value every reader of `states` sees
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w}, wh[4] = {hi.x, hi.y, hi.z, hi.w};
            const float2 a2 = unpack_x2(wl[e]), b2 = unpack_x2(wh[e]);
            cst[16 * qq + 2 * e] = a2.x; cst[16 * qq + 2 * e + 1] = a2.y;
            cst[16 * qq + 8 + 2 * e] = b2.x; cst[16 * qq + 8 + 2 * e + 1] = b2.y;
          }
        } else {
          float cv[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) cv[j] = cst[16 * qq + j];
          pack16(cv, out[0][2 * qq], out[0][2 * qq + 1]);
        }
        pack16(gi, out[1][2 * qq], out[1][2 * qq + 1]);
        pack16(gf, out[2][2 * qq], out[2][2 * qq + 1]);
        pack16(gz, out[3][2 * qq], out[3][2 * qq + 1]);
        pack16(go, out[4][2 * qq], out[4][2 * qq + 1]);
      }
      // h_t is complete: hand it to the next step first; the 20 global stores of this thread (c_t and the cache, 80 KB per
      // step and CTA) come after the arrival, off the chain h_t -> MMA -> accumulator (LB forward loop 2.87 -> 2.63 ms
      // together with the 32-byte stores).
      fence_proxy_async_smem();  // the tile is read by the tensor core and by the bulk store
      tc_fence_before();
      mbar_arrive(h_ready);
      // A thread owns 64 contiguous bytes per value kind.  Neighbouring lanes (rows 2m, 2m+1) swap halves so that each of
      // the two store instructions covers 16 rows x 64 contiguous bytes instead of 32 rows x 32: the memory system is
      // charged per piece of a 128-byte line, and this halves the pieces.
#pragma unroll
      for (int k = GRU ? 1 : 0; k < 1 + WL_G; ++k) {  // (the GRU has no second state)
        if (k > 0 && ch_e == nullptr) break;
        const uint4 s0 = odd ? out[k][0] : out[k][2], s1 = odd ? out[k][1] : out[k][3];
        uint4 r0, r1;
        r0.x = __shfl_xor_sync(0xffffffffu, s0.x, 1); r0.y = __shfl_xor_sync(0xffffffffu, s0.y, 1);
        r0.z = __shfl_xor_sync(0xffffffffu, s0.z, 1); r0.w = __shfl_xor_sync(0xffffffffu, s0.w, 1);
        r1.x = __shfl_xor_sync(0xffffffffu, s1.x, 1); r1.y = __shfl_xor_sync(0xffffffffu, s1.y, 1);
        r1.z = __shfl_xor_sync(0xffffffffu, s1.z, 1); r1.w = __shfl_xor_sync(0xffffffffu, s1.w, 1);
        void* de = k == 0 ? static_cast<void*>(c_e) : static_cast<void*>(ch_e + 512 * (k - 1));
        void* dn = k == 0 ? static_cast<void*>(c_o) : static_cast<void*>(ch_o + 512 * (k - 1));
        if (ok_e) st_global_32B(de, odd ? r0 : out[k][0], odd ? r1 : out[k][1]);
        if (ok_o) st_global_32B(dn, odd ? out[k][2] : r0, odd ? out[k][3] : r1);
      }
      c_e += ND; c_o += ND;
      if (ch_e != nullptr) { ch_e += ch_step; ch_o += ch_step; }

    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}


// ================================================================================================ backward
struct WideBwdParams {
  const elem_t* R;  // [1,N,64,64]
  elem_t* ds0;      // [1,B,1,N,64]
  float* dR;               // fp32 [1,N,64,64], accumulated with atomics
  float* dbias;            // fp32 [1,N,64]
  unsigned* status;
  int B, T, N;
  int test_drop;  // test hook: the copy of one tile (step index 2) is announced to its barrier but never issued
};

constexpr uint32_t WB_OFF_H = 0;                                  // h tiles: sequence index q <-> time T-1-q (q = T: h_{-1})
constexpr uint32_t WB_OFF_E = WB_OFF_H + WB_STAGES * WTILE;       // cotangent tiles: sequence index j <-> time T-1-j
constexpr uint32_t WB_OFF_D = WB_OFF_E + WB_STAGES * WTILE;       // delta tiles: step index j in tile j % 3, or (PAIR) time t in
                                                                  // slot t & 1 of two-step buffer (t >> 1) & 1
constexpr uint32_t WB_OFF_R = WB_OFF_D + 4 * WTILE;               // R as [p][d] (K-major B operand of delta * R)
constexpr uint32_t WB_OFF_I = WB_OFF_R + WMAT;
constexpr uint32_t WB_OFF_DB = WB_OFF_I + WMAT;                   // float[4][64]: per-warp sums of db
constexpr uint32_t WB_OFF_BAR = WB_OFF_DB + 1024;
constexpr uint32_t WB_SMEM = WB_OFF_BAR + 8 * (2 * WB_STAGES + 8) + 16 + 1024;

// PAIR: two time steps per bulk copy (maps of map_pairs, see the forward kernel).  The deltas of times 2p, 2p+1 leave in
// one store from slot time & 1 of buffer p & 1; box r of the h sequence and of the cotangent sequence holds times 2p, 2p+1
// with p = P-1-r (P = ceil(T/2)) in slot time & 1 of buffer r & 1, and box P of the h sequence is h_{-1} (one tile, plain
// layout).  A buffer goes back to the copy engine once the MMAs that read it have signalled h_free / e_free.
template <bool PAIR>
__global__ void __launch_bounds__(W_THREADS, 1)
wide_bwd_elman_kernel(const __grid_constant__ CUtensorMap tm_states, const __grid_constant__ CUtensorMap tm_s0,
                      const __grid_constant__ CUtensorMap tm_dstates, const __grid_constant__ CUtensorMap tm_dwx,
                      const WideBwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_raw + (base - raw);
  float* sdb = reinterpret_cast<float*>(sm + WB_OFF_DB);
  uint64_t* h_full = reinterpret_cast<uint64_t*>(sm + WB_OFF_BAR);  // [WB_STAGES]
  uint64_t* e_full = h_full + WB_STAGES;                            // [WB_STAGES]
  uint64_t* acc_full = e_full + WB_STAGES;                          // [2]
  uint64_t* d_ready = acc_full + 2;                                 // 128 arrivals: delta tile written
  uint64_t* dr_done = d_ready + 1;                                  // all dR MMAs have completed
  uint64_t* h_free = dr_done + 1;                                   // [2] PAIR: the MMAs that read h buffer x have completed
  uint64_t* e_free = h_free + 2;                                    // [2] PAIR: ... cotangent buffer x ...
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(e_free + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.y, b0 = blockIdx.x * WM, T = p.T;

  {
    const elem_t* Rn = p.R + (size_t)n * WD * WD;
    for (int c = tid; c < WD * 8; c += W_THREADS) {
      const uint32_t pp = c >> 3, j = c & 7;  // row p, chunk of d = 8j .. 8j+7:  Rk[p][d] = R[d][p]
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = elem_bits(Rn[(j * 8 + 2 * i) * WD + pp]);
        const uint32_t hi = elem_bits(Rn[(j * 8 + 2 * i + 1) * WD + pp]);
        w[i] = lo | (hi << 16);
      }
      *reinterpret_cast<uint4*>(sm + WB_OFF_R + sw128(pp, j)) = make_uint4(w[0], w[1], w[2], w[3]);
      const uint32_t wi = (pp & 7) >> 1, one = ((pp >> 3) == j) ? (kOneBits << (16 * (pp & 1))) : 0u;
      *reinterpret_cast<uint4*>(sm + WB_OFF_I + sw128(pp, j)) =
          make_uint4(wi == 0 ? one : 0u, wi == 1 ? one : 0u, wi == 2 ? one : 0u, wi == 3 ? one : 0u);
    }
  }
  if (tid == 0) {
    for (int s = 0; s < WB_STAGES; ++s) { mbar_init(&h_full[s], 1); mbar_init(&e_full[s], 1); }
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_full[1], 1);
    mbar_init(d_ready, WM);
    mbar_init(dr_done, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&h_free[s], 1); mbar_init(&e_free[s], 1); }
    fence_mbar_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, 256);  // columns [0,128): two dh accumulators; [128,192): dR
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer
      const uint32_t idesc_kk = instr_desc_16(WM, WD, 0, 0);  // dh: [128 b] x [64 p], K = d
      const uint32_t idesc_mm = instr_desc_16(WD, WD, 1, 1);  // dR: [64 d] x [64 p], K = b; both operands MN-major
      const void* tmh = &tm_states;
      const void* tm0 = &tm_s0;
      const void* tme = &tm_dstates;
      const void* tmd = &tm_dwx;
      if constexpr (PAIR) {
        constexpr uint32_t HI = desc_hi(1024, true), HI2 = desc_hi(2048, true), PAIR16 = (2 * WTILE) >> 4;
        const uint32_t hr_lo = (base + WB_OFF_H) >> 4, er_lo = (base + WB_OFF_E) >> 4, d_lo = (base + WB_OFF_D) >> 4,
                       r_lo = (base + WB_OFF_R) >> 4, i_lo = (base + WB_OFF_I) >> 4;
        const int P = (T + 1) >> 1, bh = b0 >> 3;
        int h_loads = 0, h_seen = 0, e_loads = 0, e_seen = 0;  // boxes requested / known to have landed
        auto load_h = [&](int r) {
          const int s = r & 1;
          if (r < P) {
            mbar_arrive_expect_tx(&h_full[s], 2 * WTILE);
            tma_load_5d(base + WB_OFF_H + s * 2 * WTILE, tmh, 0, 0, 2 * (P - 1 - r), bh, n, &h_full[s]);
          } else {
            mbar_arrive_expect_tx(&h_full[s], WTILE);
            tma_load_5d(base + WB_OFF_H + s * 2 * WTILE, tm0, 0, n, 0, b0, 0, &h_full[s]);
          }
          ++h_loads;
        };
        auto load_e = [&](int r) {
          const int s = r & 1;
          mbar_arrive_expect_tx(&e_full[s], 2 * WTILE);
          if (!(p.test_drop && r == 1)) tma_load_5d(base + WB_OFF_E + s * 2 * WTILE, tme, 0, 0, 2 * (P - 1 - r), bh, n, &e_full[s]);
          ++e_loads;
        };
        auto wait_h = [&](int r) {
          if (r < h_seen) return true;
          if (!mbar_wait_bounded(&h_full[r & 1], (uint32_t)((r >> 1) & 1))) return false;
          h_seen = r + 1;
          return true;
        };
        auto wait_e = [&](int r) {
          if (r < e_seen) return true;
          if (!mbar_wait_bounded(&e_full[r & 1], (uint32_t)((r >> 1) & 1))) return false;
          e_seen = r + 1;
          return true;
        };
        int e_reload = -1;  // cotangent box whose last tile went into an accumulator during the previous iteration
        auto issue_pre = [&](int j) {  // acc[j & 1] = dh_ext(time T-1-j) * I
          const int te = T - 1 - j, r = P - 1 - (te >> 1);
          const uint32_t a = er_lo + (uint32_t)(r & 1) * PAIR16 + (uint32_t)(te & 1) * 64u, d = tmem + (j & 1) * WD;
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI2, i_lo + 2 * k, HI, idesc_kk, k);
          if (!(te & 1)) {  // both tiles of the box are consumed once these MMAs complete
            umma_commit(&e_free[r & 1]);
            e_reload = r;
          }
        };
        auto reload_e = [&]() {  // hand the buffer of a consumed box to the box two ahead
          if (e_reload < 0) return true;
          if (!mbar_wait_bounded(&e_free[e_reload & 1], (uint32_t)((e_reload >> 1) & 1))) return false;
          if (e_reload + 2 < P) load_e(e_reload + 2);
          e_reload = -1;
          return true;
        };
        load_h(0);
        load_h(1);  // box P (h_{-1}) when T <= 2
        load_e(0);
        if (P > 1) load_e(1);
        bool ok = true;
        int where = 0;
        // T odd: h box 0 holds h_{T-1} only, which no MMA reads; give its buffer the completion the later boxes get
        if (T & 1) umma_commit(&h_free[0]);
        do {
          if (!wait_e(0)) { ok = false; break; }
          issue_pre(0);
          umma_commit(&acc_full[0]);  // step 0 (t = T-1) has no recurrent part
          if (T > 1) {
            if (!wait_e(P - 1 - ((T - 2) >> 1))) { ok = false; break; }
            issue_pre(1);
          }
          for (int j = 0; j < T; ++j) {
            where = j;
            if (!mbar_wait_bounded(d_ready, (uint32_t)(j & 1))) { ok = false; break; }
            tc_fence_after();
            const int tt = T - 1 - j;  // time of step index j
            // time tt-1 lands where time tt+3 was: stored at time tt+3 (tt odd, one younger store) or tt+2 (the youngest)
            if (tt & 1) bulk_wait_group_read<1>();
            else bulk_wait_group_read<0>();
            const uint32_t dbuf = (uint32_t)((tt >> 1) & 1) * 2 * WTILE;
            const uint32_t dt = base + WB_OFF_D + dbuf, dl = d_lo + (dbuf >> 4) + (uint32_t)(tt & 1) * 64u;
            // dh accumulator of step j+1 (+)= delta_j * R; step T (the cotangent of h_{-1}) has no external part
            const uint32_t acc = tmem + ((j + 1) & 1) * WD;
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)
              umma_parts(acc, dl + 2 * k, HI2, r_lo + 2 * k, HI, idesc_kk, (j + 1 < T || k > 0) ? 1u : 0u);
            umma_commit(&acc_full[(j + 1) & 1]);
            if (!(tt & 1)) {  // deltas of times tt, tt+1 -> dWx[b0.., tt .. tt+1, 0, n, :] (tt = T-1: the second tile is clipped)
              tma_store_5d(tmd, dt, 0, 0, tt, bh, n);
              bulk_commit_group();
              // the h box of times tt, tt+1: its row threads are done (step j), and so are the dR MMAs that read it (the
              // last ones were issued in iteration j-1 and committed to h_free)
              const int r = P - 1 - (tt >> 1);
              if (!mbar_wait_bounded(&h_free[r & 1], (uint32_t)((r >> 1) & 1))) { ok = false; break; }
              if (r + 2 <= P) load_h(r + 2);
            }
            // the cotangent box consumed during the previous iteration goes back to the copy engine before anything below
            // can wait for data
            if (!reload_e()) { ok = false; break; }
            // dR += delta_j^T * h_{tt-1}
            const int rq = tt >= 1 ? P - 1 - ((tt - 1) >> 1) : P;
            if (!wait_h(rq)) { ok = false; break; }
            if (tt >= 1) {
              const uint32_t hl = hr_lo + (uint32_t)(rq & 1) * PAIR16 + (uint32_t)((tt - 1) & 1) * 64u;
#pragma unroll
              for (uint32_t ks = 0; ks < 8; ++ks)  // 16 batch rows = two 8-row groups, 4096 bytes apart per k-step
                umma_parts(tmem + 2 * WD, dl + 256 * ks, HI2, hl + 256 * ks, HI2, idesc_mm, (j > 0 || ks > 0) ? 1u : 0u);
              if (!((tt - 1) & 1)) umma_commit(&h_free[rq & 1]);  // that was the last read of the box by an MMA
            } else {
              const uint32_t hl = hr_lo + (uint32_t)(rq & 1) * PAIR16;
#pragma unroll
              for (uint32_t ks = 0; ks < 8; ++ks)
                umma_parts(tmem + 2 * WD, dl + 256 * ks, HI2, hl + 128 * ks, HI, idesc_mm, (j > 0 || ks > 0) ? 1u : 0u);
            }
            if (j + 2 < T) {
              if (!wait_e(P - 1 - ((tt - 2) >> 1))) { ok = false; break; }
              issue_pre(j + 2);
            }
          }
        } while (false);
        if (!ok) report_timeout(p.status, where);
        umma_commit(dr_done);
        for (int i = (h_seen > h_loads - 2 ? h_seen : h_loads - 2); i < h_loads; ++i)
          mbar_wait_bounded(&h_full[i & 1], (uint32_t)((i >> 1) & 1));
        for (int i = (e_seen > e_loads - 2 ? e_seen : e_loads - 2); i < e_loads; ++i)
          mbar_wait_bounded(&e_full[i & 1], (uint32_t)((i >> 1) & 1));
        bulk_wait_group<0>();
      } else {
      int h_loads = 0, h_seen = 0, e_loads = 0, e_seen = 0;  // tiles requested / known to have landed, in sequence order
      auto load_h = [&](int q) {
        const int s = q % WB_STAGES;
        mbar_arrive_expect_tx(&h_full[s], WTILE);
        if (q < T) tma_load_5d(base + WB_OFF_H + s * WTILE, tmh, 0, n, T - 1 - q, b0, 0, &h_full[s]);
        else tma_load_5d(base + WB_OFF_H + s * WTILE, tm0, 0, n, 0, b0, 0, &h_full[s]);
        ++h_loads;
      };
      auto load_e = [&](int j) {
        const int s = j % WB_STAGES;
        mbar_arrive_expect_tx(&e_full[s], WTILE);
        if (!(p.test_drop && j == 2)) tma_load_5d(base + WB_OFF_E + s * WTILE, tme, 0, n, T - 1 - j, b0, 0, &e_full[s]);
        ++e_loads;
      };
      constexpr uint32_t HI = desc_hi(1024, true), TILE16 = WTILE >> 4;  // descriptor halves as in the forward kernel
      const uint32_t hr_lo = (base + WB_OFF_H) >> 4, er_lo = (base + WB_OFF_E) >> 4, d_lo = (base + WB_OFF_D) >> 4,
                     r_lo = (base + WB_OFF_R) >> 4, i_lo = (base + WB_OFF_I) >> 4;
      auto issue_pre = [&](int j) {  // acc[j & 1] = dh_ext_j * I
        const uint32_t a = er_lo + (j % WB_STAGES) * TILE16, d = tmem + (j & 1) * WD;
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) umma_parts(d, a + 2 * k, HI, i_lo + 2 * k, HI, idesc_kk, k);
      };
      for (int q = 0; q <= T && q < WB_STAGES; ++q) load_h(q);
      for (int j = 0; j < T && j < WB_STAGES; ++j) load_e(j);
      bool ok = true;
      int where = 0;
      int dj = 0;  // delta tile of step index j
      do {
        if (!mbar_wait_bounded(&e_full[0], 0)) { ok = false; break; }
        e_seen = 1;
        issue_pre(0);
        umma_commit(&acc_full[0]);  // step 0 (t = T-1) has no recurrent part
        if (T > 1) {
          if (!mbar_wait_bounded(&e_full[1], 0)) { ok = false; break; }
          e_seen = 2;
          issue_pre(1);
        }
        for (int j = 0; j < T; ++j) {
          where = j;
          if (!mbar_wait_bounded(d_ready, (uint32_t)(j & 1))) { ok = false; break; }
          tc_fence_after();
          if (h_seen < j + 1) h_seen = j + 1;  // the row threads of step j have read h tile j
          // step j+1 overwrites the tile of delta_{j-2}: that store (two groups back) must have left shared memory
          bulk_wait_group_read<1>();
          const uint32_t dt = base + WB_OFF_D + dj * WTILE, dl = d_lo + dj * TILE16;
          // dh accumulator of step j+1 (+)= delta_j * R; step T (the cotangent of h_{-1}) has no external part
          const uint32_t acc = tmem + ((j + 1) & 1) * WD;
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k)
            umma_parts(acc, dl + 2 * k, HI, r_lo + 2 * k, HI, idesc_kk, (j + 1 < T || k > 0) ? 1u : 0u);
          umma_commit(&acc_full[(j + 1) & 1]);
          tma_store_5d(tmd, dt, 0, n, 0, T - 1 - j, b0);  // delta_j -> dWx[b0.., t, 0, n, :]
          bulk_commit_group();
          // dR += delta_j^T * h_{t-1}  (h tile of sequence index j + 1)
          if (!mbar_wait_bounded(&h_full[(j + 1) % WB_STAGES], (uint32_t)(((j + 1) / WB_STAGES) & 1))) { ok = false; break; }
          h_seen = j + 2;
          const uint32_t hl = hr_lo + ((j + 1) % WB_STAGES) * TILE16;
#pragma unroll
          for (uint32_t ks = 0; ks < 8; ++ks)  // 16 batch rows = 2048 bytes per k-step
            umma_parts(tmem + 2 * WD, dl + 128 * ks, HI, hl + 128 * ks, HI, idesc_mm, (j > 0 || ks > 0) ? 1u : 0u);
          // h tile j-1: its row threads (step j-1) and its dR MMAs (step j-2, completed before the accumulator of
          // step j was signalled) are done; cotangent tile j: consumed by MMAs that completed before step j started
          if (j >= 1 && j - 1 + WB_STAGES <= T) load_h(j - 1 + WB_STAGES);
          if (j + WB_STAGES < T) load_e(j + WB_STAGES);
          if (j + 2 < T) {
            if (!mbar_wait_bounded(&e_full[(j + 2) % WB_STAGES], (uint32_t)(((j + 2) / WB_STAGES) & 1))) { ok = false; break; }
            e_seen = j + 3;
            issue_pre(j + 2);
          }
          dj = (dj == 2) ? 0 : dj + 1;
        }
      } while (false);
      if (!ok) report_timeout(p.status, where);
      umma_commit(dr_done);
      for (int i = (h_seen > h_loads - WB_STAGES ? h_seen : h_loads - WB_STAGES); i < h_loads; ++i)
        mbar_wait_bounded(&h_full[i % WB_STAGES], (uint32_t)((i / WB_STAGES) & 1));
      for (int i = (e_seen > e_loads - WB_STAGES ? e_seen : e_loads - WB_STAGES); i < e_loads; ++i)
        mbar_wait_bounded(&e_full[i % WB_STAGES], (uint32_t)((i / WB_STAGES) & 1));
      bulk_wait_group<0>();
      }
    }
  } else {
    // ------------------------------------------------------------ row threads: delta_t = dh_t * (1 - h_t^2)
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    float db[WD];
#pragma unroll
    for (int i = 0; i < WD; ++i) db[i] = 0.f;
    bool ok = true;
    int dw = 0;  // tile that receives delta of step index j
    for (int j = 0; j < T; ++j) {
      const int tt = T - 1 - j, hr = ((T + 1) >> 1) - 1 - (tt >> 1);  // time of the step; PAIR: its h box
      if (!mbar_wait_bounded(&acc_full[j & 1], (uint32_t)((j >> 1) & 1)) ||
          !(PAIR ? mbar_wait_bounded(&h_full[hr & 1], (uint32_t)((hr >> 1) & 1))
                  : mbar_wait_bounded(&h_full[j % WB_STAGES], (uint32_t)((j / WB_STAGES) & 1)))) {
        report_timeout(p.status, j);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld64(trow + (j & 1) * WD, r0, r1);
      const unsigned char* hsrc = sm + WB_OFF_H + (PAIR ? (uint32_t)(hr & 1) * 2 * WTILE : (j % WB_STAGES) * WTILE);
      unsigned char* dst = sm + WB_OFF_D + (PAIR ? (uint32_t)((tt >> 1) & 1) * 2 * WTILE : dw * WTILE);
      dw = (dw == 2) ? 0 : dw + 1;
#pragma unroll
      for (uint32_t c = 0; c < 8; ++c) {
        const uint32_t off = sw128(tid, c);
        const uint4 hv = *reinterpret_cast<const uint4*>(hsrc + (PAIR ? sw128_pair(tid, c, tt & 1) : off));
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 h2 = unpack_x2(hw[i]);
          const float g0 = __uint_as_float(c < 4 ? r0[c * 8 + 2 * i] : r1[(c - 4) * 8 + 2 * i]);
          const float g1 = __uint_as_float(c < 4 ? r0[c * 8 + 2 * i + 1] : r1[(c - 4) * 8 + 2 * i + 1]);
          v[2 * i] = g0 * (1.f - h2.x * h2.x);
          v[2 * i + 1] = g1 * (1.f - h2.y * h2.y);
          db[c * 8 + 2 * i] += v[2 * i];
          db[c * 8 + 2 * i + 1] += v[2 * i + 1];
        }
        *reinterpret_cast<uint4*>(dst + (PAIR ? sw128_pair(tid, c, tt & 1) : off)) = pack8(v);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(d_ready);
    }
    // cotangent of the initial state: the accumulator of "step T"
    if (ok && mbar_wait_bounded(&acc_full[T & 1], (uint32_t)((T >> 1) & 1))) {
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld64(trow + (T & 1) * WD, r0, r1);
      const int b = b0 + tid;
      if (b < p.B) {
        uint4* out = reinterpret_cast<uint4*>(p.ds0 + ((size_t)b * p.N + n) * WD);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(c < 4 ? r0[c * 8 + i] : r1[(c - 4) * 8 + i]);
          out[c] = pack8(v);
        }
      }
    } else if (ok) {
      report_timeout(p.status, T);
      ok = false;
    }
    // dR: row d of the 64 x 64 accumulator sits in lane (d / 16) * 32 + d % 16 of tensor memory
    if (ok && mbar_wait_bounded(dr_done, 0)) {
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld64(trow + 2 * WD, r0, r1);
      if (lane < 16) {
        float* out = p.dR + ((size_t)n * WD + (warp * 16 + lane)) * WD;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          red_add_f32x4(out + i, __uint_as_float(r0[i]), __uint_as_float(r0[i + 1]), __uint_as_float(r0[i + 2]),
                        __uint_as_float(r0[i + 3]));
          red_add_f32x4(out + 32 + i, __uint_as_float(r1[i]), __uint_as_float(r1[i + 1]), __uint_as_float(r1[i + 2]),
                        __uint_as_float(r1[i + 3]));
        }
      }
    } else if (ok) {
      report_timeout(p.status, T + 1);
    }
#pragma unroll
    for (int i = 0; i < WD; ++i) {  // db: sum over the 32 rows of the warp by shuffles, then one partial per warp
      float v = db[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) sdb[warp * WD + i] = v;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid < WD) atomicAdd(p.dbias + (size_t)n * WD + tid, sdb[tid] + sdb[WD + tid] + sdb[2 * WD + tid] + sdb[3 * WD + tid]);
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, 256);
  }
}

// ================================================================================================ host
// tiles of 64 elements x 128 entries of dimension `batch_dim` of a bf16 tensor seen as 5-d
bool encode_tiles(CUtensorMap* tm, const void* base, const uint64_t (&dims)[5], const uint64_t (&strides)[4], int batch_dim) {
  uint32_t box[5] = {WD, 1, 1, 1, 1};
  box[batch_dim] = WM;
  return encode_tiles16(tm, base, dims, strides, box);
}

// Element strides of the batch, time and head dimensions of a tensor whose head dim (64 elements) is contiguous.
struct RowStrides { long long sb, st, sn; };
static RowStrides dense_strides(int T, int N) { return RowStrides{(long long)T * N * WD, (long long)N * WD, WD}; }

// [B,T,1,N,64] (Wx, dWx): coordinates (0, n, 0, t, b)
bool map_btgnd(CUtensorMap* tm, const void* base, int B, int T, int N, RowStrides s) {
  const uint64_t dims[5] = {WD, (uint64_t)N, 1, (uint64_t)T, (uint64_t)B};
  const uint64_t strides[4] = {(uint64_t)s.sn * 2, (uint64_t)s.st * 2, (uint64_t)s.st * 2, (uint64_t)s.sb * 2};
  return encode_tiles(tm, base, dims, strides, 4);
}
// [1,B,T,N,64] (states, dstates): coordinates (0, n, t, b, 0);  T = 1 gives the initial-state layout [1,B,1,N,64]
bool map_sbtnd(CUtensorMap* tm, const void* base, int B, int T, int N, RowStrides s) {
  const uint64_t dims[5] = {WD, (uint64_t)N, (uint64_t)T, (uint64_t)B, 1};
  const uint64_t strides[4] = {(uint64_t)s.sn * 2, (uint64_t)s.st * 2, (uint64_t)s.sb * 2, (uint64_t)s.sb * 2};
  return encode_tiles(tm, base, dims, strides, 3);
}

// Both layouts ([B,T,1,N,64] and [1,B,T,N,64]) with B a multiple of 8, two time steps per box: coordinates
// (0, 0, t, b / 8, n); a box is [16 groups of 8 rows][2 steps][8 rows][64], so each group's pages are touched twice in a row
bool map_pairs(CUtensorMap* tm, const void* base, int B, int T, int N, RowStrides s) {
  const uint64_t dims[5] = {WD, 8, (uint64_t)T, (uint64_t)B / 8, (uint64_t)N};
  const uint64_t strides[4] = {(uint64_t)s.sb * 2, (uint64_t)s.st * 2, (uint64_t)s.sb * 16, (uint64_t)s.sn * 2};
  const uint32_t box[5] = {WD, 8, 2, WM / 8, 1};
  return encode_tiles16(tm, base, dims, strides, box);
}
bool pairs_ok(int B, int T) { return B % 8 == 0 && T >= 2; }

// Wx [B,T,4,N,64] seen as (d, b, g, n, t): one box [4 gates][128 rows][64] per (tile, head, step)
bool map_wx_gates(CUtensorMap* tm, const void* base, int gates, int B, int T, int N, long long sb, long long st, long long sg,
                  long long sn) {
  const uint64_t dims[5] = {WD, (uint64_t)B, (uint64_t)gates, (uint64_t)N, (uint64_t)T};
  const uint64_t strides[4] = {(uint64_t)sb * 2, (uint64_t)sg * 2, (uint64_t)sn * 2, (uint64_t)st * 2};
  const uint32_t box[5] = {WD, WM, (uint32_t)gates, 1, 1};
  return encode_tiles16(tm, base, dims, strides, box);
}

}  // namespace

bool wide_supported(int cell, int D, int state_f32, float fclip, float gclip, int grad_cut) {
  return cell == CELL_ELMAN && D == WD && !state_f32 && !(fclip > 0.f) && !(gclip > 0.f) && !grad_cut;
}

cudaError_t launch_wide_forward(const void* Wx, long long wx_sb, long long wx_st, long long wx_sn, const void* R,
                                const void* bias, const void* s0, void* states, unsigned* status, int B, int T, int N,
                                int test_drop, cudaStream_t stream) {
  CUtensorMap tm_wx, tm_st;
  const bool pair = pairs_ok(B, T);
  const RowStrides dense = dense_strides(T, N), wxs = RowStrides{wx_sb, wx_st, wx_sn};
  if (pair ? (!map_pairs(&tm_wx, Wx, B, T, N, wxs) || !map_pairs(&tm_st, states, B, T, N, dense))
           : (!map_btgnd(&tm_wx, Wx, B, T, N, wxs) || !map_sbtnd(&tm_st, states, B, T, N, dense)))
    return cudaErrorNotSupported;
  WideFwdParams p;
  p.R = static_cast<const elem_t*>(R);
  p.bias = static_cast<const elem_t*>(bias);
  p.s0 = static_cast<const elem_t*>(s0);
  p.status = status;
  p.B = B; p.T = T; p.N = N;
  p.test_drop = test_drop;
  auto kern = pair ? wide_fwd_elman_kernel<true> : wide_fwd_elman_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WF_SMEM);
  if (e != cudaSuccess) return e;
  kern<<<dim3((unsigned)((B + WM - 1) / WM), (unsigned)N), W_THREADS, WF_SMEM, stream>>>(tm_wx, tm_st, p);
  return cudaGetLastError();
}

// 128-row forward loop of the LSTM and GRU cells at head dim 64 (16-bit states); the reverse loop stays
// on the cluster kernels' 16-row tiles, whose cache layout the forward loop writes
bool wide_gates_forward_supported(int cell, int D, int state_f32) {
  return (cell == CELL_LSTM || cell == CELL_GRU) && D == WD && !state_f32;
}

cudaError_t launch_wide_gates_forward(int cell, const void* Wx, long long wx_sb, long long wx_st, long long wx_sg, long long wx_sn, const void* R,
                                     const void* bias, const void* s0, void* states, void* cache, unsigned* status, int B, int T,
                                     int N, float fclip, int test_drop, cudaStream_t stream) {
  CUtensorMap tm_wx, tm_st;
  if (!map_wx_gates(&tm_wx, Wx, cell == CELL_GRU ? 3 : 4, B, T, N, wx_sb, wx_st, wx_sg, wx_sn) ||
      !map_sbtnd(&tm_st, states, B, T, N, dense_strides(T, N)))
    return cudaErrorNotSupported;
  WideGatesParams p;
  p.R = static_cast<const elem_t*>(R);
  p.bias = static_cast<const elem_t*>(bias);
  p.s0 = static_cast<const elem_t*>(s0);
  p.states = static_cast<elem_t*>(states);
  p.cache = static_cast<uint32_t*>(cache);
  p.status = status;
  p.B = B; p.T = T; p.N = N;
  p.test_drop = test_drop;
  p.fclip = fclip;
  auto kern = cell == CELL_GRU ? wide_fwd_gates_kernel<CELL_GRU> : wide_fwd_gates_kernel<CELL_LSTM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WL_SMEM);
  if (e != cudaSuccess) return e;
  kern<<<dim3((unsigned)((B + WM - 1) / WM), (unsigned)N), WL_THREADS, WL_SMEM, stream>>>(tm_wx, tm_st, p);
  return cudaGetLastError();
}

cudaError_t launch_wide_backward(const void* R, const void* s0, const void* states, const void* dstates, long long ds_sb,
                                 long long ds_st, long long ds_sn, void* dWx, void* ds0, float* dR, float* dbias,
                                 unsigned* status, int B, int T, int N, int test_drop, cudaStream_t stream) {
  CUtensorMap tm_st, tm_s0, tm_dst, tm_dwx;
  const bool pair = pairs_ok(B, T);
  const RowStrides dense = dense_strides(T, N), dss = RowStrides{ds_sb, ds_st, ds_sn};
  if (!(pair ? map_pairs(&tm_st, states, B, T, N, dense) : map_sbtnd(&tm_st, states, B, T, N, dense)) ||
      !map_sbtnd(&tm_s0, s0, B, 1, N, dense_strides(1, N)) ||
      !(pair ? map_pairs(&tm_dst, dstates, B, T, N, dss) : map_sbtnd(&tm_dst, dstates, B, T, N, dss)) ||
      !(pair ? map_pairs(&tm_dwx, dWx, B, T, N, dense) : map_btgnd(&tm_dwx, dWx, B, T, N, dense)))
    return cudaErrorNotSupported;
  WideBwdParams p;
  p.R = static_cast<const elem_t*>(R);
  p.ds0 = static_cast<elem_t*>(ds0);
  p.dR = dR;
  p.dbias = dbias;
  p.status = status;
  p.B = B; p.T = T; p.N = N;
  p.test_drop = test_drop;
  auto kern = pair ? wide_bwd_elman_kernel<true> : wide_bwd_elman_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WB_SMEM);
  if (e != cudaSuccess) return e;
  kern<<<dim3((unsigned)((B + WM - 1) / WM), (unsigned)N), W_THREADS, WB_SMEM, stream>>>(tm_st, tm_s0, tm_dst,
                                                                                                          tm_dwx, p);
  return cudaGetLastError();
}

}  // namespace FRNN_NS
