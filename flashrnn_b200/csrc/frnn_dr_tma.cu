// dR on the 5th-generation tensor cores, operands fetched by tensor-map bulk copies.
//
//   dR[g,n,d,p] = sum_{b,t} delta_g[b,t,n,d] * h_{t-1}[b,n,p]
//
// Same GEMM as frnn_dr_tc.cu (C[(g,d), p] = A^T B per head, both operands MN-major exactly as the time loops left them
// in HBM), for bf16 states and head dims that are multiples of 64: a 64-step stretch of one batch row is, for every 64
// consecutive d (or p), one [64 t][64] tile with 128-byte rows -- the box of a tensor-map copy with 128-byte swizzle
// and, unchanged, one block of a UMMA operand.  One CTA owns MT tiles of 128 rows of (g,d) (two such blocks each), all D
// columns of p and a range of 64-step chunks (split-K over gridDim.z); the MT accumulators share every h block that is
// fetched, so h crosses L2 -> shared memory once per MT * 128 rows (MT = 2 for D = 256, 3 for D = 128: the tensor
// memory holds MT * D <= 512 fp32 columns):
//   * warp 4, one lane: per chunk 2 MT + D/64 bulk loads into a 3- or 4-stage ring (mbarrier byte counts), then 4 MT
//     tcgen05.mma (M128, N = D, K16) accumulating in tensor memory; tcgen05.commit frees the stage;
//   * h_{t-1} of t = 0 is the initial state, which is not a row of `states`: the copy starts at t = -1, that row reads
//     as zero, and the missing products delta[b,0] * h_{-1}[b] are added by the draining threads from global memory;
//   * warps 0-3 read their tensor-memory lanes and add the tile into the fp32 gradient workspace with atomics.
// Every wait is bounded; on expiry the CTA records it, stops issuing and waits (bounded) for the copies in flight.
//
// Replaces the post-loop cublasGemmStridedBatchedEx of the reference (flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:
// 1049-1058; util/blas.cu:199-219).
#include "frnn_aux.cuh"
#include "frnn_tc.cuh"
#include "frnn_tmap.cuh"

namespace FRNN_NS {

namespace {

constexpr int DT_KC = 64;                      // time steps per chunk = rows of a block
constexpr int DT_STAGES = 4;
constexpr int DT_THREADS = 160;                // warps 0-3 drain tensor memory; warp 4, lane 0 issues copies and MMAs
constexpr uint32_t DT_BLK = 64 * DT_KC * 2;    // bytes of one [64 t][64] bf16 block

struct DrTmaParams {
  const elem_t* dWx;  // [B,T,Gw,N,D]
  const elem_t* dg0;  // [B,T,N,D] (GRU)
  const elem_t* s0;   // [S,B,1,N,D]; only s = 0 is read
  float* dR;                 // [Gr,N,D,D] fp32
  unsigned* status;
  int cell, B, T, N, D, Gr, Gw;
  int chunks_per_b;          // ceil(T / 64)
  int chunks_per_split;
  int tmem_cols;             // power of two >= mt * D, >= 32
  int mt;                    // 128-row tiles of (g,d) per CTA
  int stages;                // ring depth (<= DT_STAGES)
};

__global__ void __launch_bounds__(DT_THREADS, 1)
recurrent_grad_tma_kernel(const __grid_constant__ CUtensorMap tm_dwx, const __grid_constant__ CUtensorMap tm_dg0,
                          const __grid_constant__ CUtensorMap tm_states, const DrTmaParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_raw + (base - raw);
  const int D = p.D, N = p.N, T = p.T, nb = D >> 6;  // nb = 64-wide blocks per gate (rows) / of p (columns)
  const int MT = p.mt, NS = p.stages;
  const uint32_t stage_bytes = (uint32_t)(2 * MT + nb) * DT_BLK;
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + (size_t)NS * stage_bytes);          // [DT_STAGES] bytes have landed
  uint64_t* empty = full + DT_STAGES;                                                  // [DT_STAGES] MMAs have read the stage
  uint64_t* done = empty + DT_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.y;
  const int RB = p.Gr * nb;                            // 64-row blocks of (g,d)
  const int rbase = 2 * MT * blockIdx.x;               // blocks rbase .. rbase + 2 MT - 1; those beyond RB repeat the last one
                                                       // (computed again, not stored)
  const long long total_chunks = (long long)p.B * p.chunks_per_b;
  const long long c_begin = (long long)blockIdx.z * p.chunks_per_split;
  long long c_end = c_begin + p.chunks_per_split;
  if (c_end > total_chunks) c_end = total_chunks;
  if (c_begin >= c_end) return;  // uniform for the CTA
  const int nchunks = (int)(c_end - c_begin);

  if (tid == 0) {
    for (int s = 0; s < DT_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(done, 1);
    fence_mbar_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc_16(128, D, 1, 1);  // both operands MN-major
      constexpr uint32_t HI = desc_hi(1024, true);
      constexpr uint32_t LBO = (DT_BLK >> 4) << 16;          // 64-wide blocks of m / n follow each other at 8 KB
      const void* tmw = &tm_dwx;
      const void* tmg = &tm_dg0;
      const void* tmh = &tm_states;
      int loads = 0, seen = 0;  // chunks requested / seen to land
      int ls = 0;               // ring stage of the next request (requests go out in chunk order)
      int lb = (int)(c_begin / p.chunks_per_b), lc = (int)(c_begin - (long long)lb * p.chunks_per_b);  // its batch row, chunk
      auto load = [&](int) {
        const int b = lb, t0 = lc * DT_KC;
        if (++lc == p.chunks_per_b) { lc = 0; ++lb; }
        const int s = ls;
        ls = (ls + 1 == NS) ? 0 : ls + 1;
        const uint32_t dst = base + (uint32_t)s * stage_bytes;
        mbar_arrive_expect_tx(&full[s], stage_bytes);
        for (int i = 0; i < 2 * MT; ++i) {
          const int rb = (rbase + i < RB) ? rbase + i : RB - 1, g = rb / nb, d0 = (rb - g * nb) * 64;
          if (p.cell == CELL_GRU && g == 0) tma_load_5d(dst + i * DT_BLK, tmg, d0, n, t0, b, 0, &full[s]);
          else tma_load_5d(dst + i * DT_BLK, tmw, d0, n, (p.cell == CELL_GRU) ? g - 1 : g, t0, b, &full[s]);
        }
        for (int pb = 0; pb < nb; ++pb) tma_load_5d(dst + (2 * MT + pb) * DT_BLK, tmh, pb * 64, n, t0 - 1, b, 0, &full[s]);
        ++loads;
      };
      for (int ci = 0; ci < nchunks && ci < NS; ++ci) load(ci);
      bool ok = true;
      int s = 0, ps = 0;         // ring stage of chunk ci and of chunk ci - 1
      uint32_t par = 0, ppar = 0;  // and the parities of their barrier phases
      for (int ci = 0; ci < nchunks; ++ci) {
        if (!mbar_wait_bounded(&full[s], par)) { ok = false; report_timeout(p.status, ci); break; }
        seen = ci + 1;
        const uint32_t s_lo = ((base + (uint32_t)s * stage_bytes) >> 4) | LBO, b_lo = s_lo + (uint32_t)MT * ((2 * DT_BLK) >> 4);
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t a_lo = s_lo + (uint32_t)mt * ((2 * DT_BLK) >> 4), acc = tmem + (uint32_t)(mt * D);
#pragma unroll
          for (uint32_t ks = 0; ks < DT_KC / 16; ++ks)  // 16 rows of a block = 2048 bytes per k-step
            umma_parts(acc, a_lo + 128 * ks, HI, b_lo + 128 * ks, HI, idesc, (ci > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        if (ci >= 1 && ci - 1 + NS < nchunks) {  // refill the stage of the chunk before: its MMAs are done sooner
          if (!mbar_wait_bounded(&empty[ps], ppar)) {
            ok = false;
            report_timeout(p.status, ci);
            break;
          }
          load(ci - 1 + NS);
        }
        ps = s; ppar = par;
        if (++s == NS) { s = 0; par ^= 1u; }
      }
      umma_commit(done);
      if (!ok)  // never leave with copies in flight
        for (int i = (seen > loads - NS ? seen : loads - NS); i < loads; ++i)
          mbar_wait_bounded(&full[i % NS], (uint32_t)((i / NS) & 1));
    }
  } else {
    // ---- drain: row m of tile mt = (block 2 mt + m / 64, d = 64 * dblk + m % 64)
    const bool fin = mbar_wait_bounded(done, 0);
    if (!fin) report_timeout(p.status, nchunks);
    tc_fence_after();
    const int m = warp * 32 + lane;
    // delta[b, t = 0] of a row is needed for the batch rows whose first chunk belongs to this CTA
    const int b_first = (int)((c_begin + p.chunks_per_b - 1) / p.chunks_per_b), b_last = (int)((c_end - 1) / p.chunks_per_b);
    const size_t ND = (size_t)N * D;
    for (int mt = 0; mt < MT; ++mt) {
    const int rb = rbase + 2 * mt + (m >> 6);
    const bool row_ok = fin && rb < RB;
    const int rbc = row_ok ? rb : RB - 1, g = rbc / nb, d = (rbc - g * nb) * 64 + (m & 63);
    float* out = p.dR + (((size_t)g * N + n) * D + d) * D;
    const bool from_dg0 = p.cell == CELL_GRU && g == 0;
    const elem_t* d0src = from_dg0 ? p.dg0 + (size_t)n * D + d
                                          : p.dWx + (size_t)((p.cell == CELL_GRU) ? g - 1 : g) * ND + (size_t)n * D + d;
    const size_t d0stride = (from_dg0 ? (size_t)1 : (size_t)p.Gw) * ND * T;  // elements between batch rows at t = 0
    for (int col0 = 0; col0 < D; col0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(mt * D + col0), r);
      if (!row_ok) continue;
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      for (int b = b_first; b <= b_last; ++b) {  // h_{-1}: the products the zero row at t = -1 left out
        const float dv = elem_to_float(d0src[(size_t)b * d0stride]);
        const uint4* hs = reinterpret_cast<const uint4*>(p.s0 + ((size_t)b * N + n) * D + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 w = hs[q];
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 h2 = unpack_x2(ww[e]);
            v[q * 8 + 2 * e] = fmaf(dv, h2.x, v[q * 8 + 2 * e]);
            v[q * 8 + 2 * e + 1] = fmaf(dv, h2.y, v[q * 8 + 2 * e + 1]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 32; j += 4) red_add_f32x4(out + col0 + j, v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, (uint32_t)p.tmem_cols);
  }
}

}  // namespace

bool recurrent_grad_tma_supported(int D, int state_f32) { return !state_f32 && D >= 64 && D <= 256 && D % 64 == 0; }

cudaError_t launch_recurrent_grad_tma(int cell, int B, int T, int N, int D, int Gr, int Gw, const void* dWx, const void* dg0,
                                      const void* states, const void* s0, float* dR, unsigned* status, int sm_count,
                                      cudaStream_t stream) {
  const uint64_t row = (uint64_t)D * 2;
  CUtensorMap tm_dwx, tm_dg0, tm_st;
  {
    const uint64_t dims[5] = {(uint64_t)D, (uint64_t)N, (uint64_t)Gw, (uint64_t)T, (uint64_t)B};
    const uint64_t str[4] = {row, row * N, row * N * Gw, row * N * Gw * T};
    const uint32_t box[5] = {64, 1, 1, DT_KC, 1};
    if (!encode_tiles16(&tm_dwx, dWx, dims, str, box)) return cudaErrorNotSupported;
  }
  {
    // [B,T,N,D] (GRU: delta of the recurrent-only gate) and states[0] = [B,T,N,D]: coordinates (d, n, t, b, 0)
    const uint64_t dims[5] = {(uint64_t)D, (uint64_t)N, (uint64_t)T, (uint64_t)B, 1};
    const uint64_t str[4] = {row, row * N, row * N * T, row * N * T * B};
    const uint32_t box[5] = {64, 1, DT_KC, 1, 1};
    if (!encode_tiles16(&tm_dg0, cell == CELL_GRU ? dg0 : states, dims, str, box)) return cudaErrorNotSupported;
    if (!encode_tiles16(&tm_st, states, dims, str, box)) return cudaErrorNotSupported;
  }
  DrTmaParams p;
  p.dWx = static_cast<const elem_t*>(dWx);
  p.dg0 = static_cast<const elem_t*>(dg0);
  p.s0 = static_cast<const elem_t*>(s0);
  p.dR = dR;
  p.status = status;
  p.cell = cell; p.B = B; p.T = T; p.N = N; p.D = D; p.Gr = Gr; p.Gw = Gw;
  p.chunks_per_b = (T + DT_KC - 1) / DT_KC;
  // tiles of 128 rows per CTA: as many as share one fetch of h, within 512 tensor-memory columns and a ring of at least
  // three stages in shared memory
  const int nb = D / 64, tiles = (Gr * nb + 1) / 2;
  int mt = 512 / D;
  if (mt > 3) mt = 3;
  if (mt > tiles) mt = tiles;
  while (mt > 1 && 3 * (size_t)(2 * mt + nb) * DT_BLK > (size_t)200 * 1024) --mt;
  mt = (tiles + (tiles + mt - 1) / mt - 1) / ((tiles + mt - 1) / mt);  // same number of CTAs, evenly filled
#ifdef FRNN_DR_ONE_TILE  // development aid: one tile per CTA
  mt = 1;
#endif
  p.mt = mt;
  int stages = (int)(((size_t)200 * 1024) / ((size_t)(2 * mt + nb) * DT_BLK));
  p.stages = stages > DT_STAGES ? DT_STAGES : stages;
  int cols = 32;
  while (cols < mt * D) cols *= 2;
  p.tmem_cols = cols;
  const int mtiles = (tiles + mt - 1) / mt;
  const long long chunks = (long long)B * p.chunks_per_b;
  const long long base_ctas = (long long)mtiles * N;
  long long splits = sm_count / base_ctas;  // one CTA per SM (shared memory): stay within a single wave
  if (splits > (chunks + 3) / 4) splits = (chunks + 3) / 4;  // at least 4 chunks per split
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  p.chunks_per_split = (int)((chunks + splits - 1) / splits);
  splits = (chunks + p.chunks_per_split - 1) / p.chunks_per_split;
  const size_t smem = (size_t)p.stages * (2 * mt + nb) * DT_BLK + 8 * (2 * DT_STAGES + 1) + 16 + 1024;
  cudaError_t e = cudaFuncSetAttribute(recurrent_grad_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);  // fixed maximum, so that concurrent host threads never lower each other's setting
  if (e != cudaSuccess) return e;
  recurrent_grad_tma_kernel<<<dim3((unsigned)mtiles, (unsigned)N, (unsigned)splits), DT_THREADS, smem, stream>>>(tm_dwx, tm_dg0,
                                                                                                                 tm_st, p);
  return cudaGetLastError();
}

}  // namespace FRNN_NS
