// dR on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   dR[g,n,d,p] = sum_{b,t} delta_g[b,t,n,d] * h_{t-1}[b,n,p]
//
// is, per head n, one GEMM  C[(g,d), p] = A^T B  with  A[k, (g,d)] = delta rows and B[k, p] = h_{t-1} rows,
// k = b*T + t.  Both operands arrive "MN-major" (k is the slow index of the tensors the time loops wrote), which the
// UMMA shared-memory descriptors consume directly: no transposition anywhere.
//
// One CTA owns a 128-row tile of (g,d) x all D columns of p and a contiguous range of k (split-K over gridDim.z):
//   * cp.async (16 B) streams 64-row k-chunks of A and B into a 3-stage ring laid out as UMMA core matrices
//     (8 k-rows x 16 B, no swizzle);
//   * one thread issues 4 x tcgen05.mma (M128, N = D, K16, bf16 -> fp32) per chunk, accumulating in TMEM;
//     tcgen05.commit signals an mbarrier per stage so that the ring slot can be refilled;
//   * after the last chunk the 4 warps read their 32 TMEM lanes (tcgen05.ld) and add the tile into the fp32
//     gradient workspace with atomics (the k-splits and the batch shards of other calls meet there).
// Every mbarrier wait is bounded; on expiry the CTA records it in the status block and leaves the loop.
//
// Replaces the post-loop cublasGemmStridedBatchedEx of the reference (flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:
// 1049-1058; util/blas.cu:199-219).
#include "frnn_aux.cuh"
#include "frnn_tc.cuh"

namespace FRNN_NS {

namespace {

constexpr int TC_M = 128;            // rows of (g,d) per CTA = UMMA M
constexpr int TC_KC = 64;            // k rows per ring stage (4 MMAs of K = 16)
constexpr int TC_STAGES = 3;
constexpr int TC_THREADS = 256;       // 8 loader warps; warps 0-3 also drain TMEM
constexpr int TC_KG = TC_KC / 8;     // 8-row k groups per stage
constexpr int TC_LBO = 128;          // bytes between core matrices adjacent in k
constexpr int TC_SBO = TC_KG * 128 + 16;  // bytes between core matrices adjacent in (g,d) / p; +16 spreads the banks

struct DrTcParams {
  const elem_t* dWx;  // [B,T,Gw,N,D]
  const elem_t* dg0;  // [B,T,N,D] (GRU)
  const void* states;        // [S,B,T,N,D]; only s = 0 is read
  const void* s0;            // [S,B,1,N,D]
  float* dR;                 // [Gr,N,D,D] fp32
  unsigned* status;
  int cell, T, N, D, Gr, Gw, state_f32;
  long long K;               // B*T
  int chunks_per_split;
  int tmem_cols;             // power of two >= J * D, >= 32
};

size_t tc_smem_bytes(int D, int J) {
  return (size_t)TC_STAGES * ((size_t)(J * TC_M / 8) * TC_SBO + (size_t)(D / 8) * TC_SBO) + 64;
}

// J: tiles of 128 rows of (g,d) per CTA.  Their accumulators (J * D <= 512 tensor-memory columns) share every h row that
// is staged, so h is read from L2 once per J * 128 rows.
template <bool F32, int J>
__global__ void __launch_bounds__(TC_THREADS, 1) recurrent_grad_tc_kernel(const DrTcParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int D = p.D, N = p.N, T = p.T, Gr = p.Gr;
  const int mtile = blockIdx.x, n = blockIdx.y;
  const size_t ND = (size_t)N * D;
  const uint32_t a_bytes = (uint32_t)(J * TC_M / 8) * TC_SBO, b_bytes = (uint32_t)(D / 8) * TC_SBO;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)TC_STAGES * stage_bytes);  // [TC_STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + TC_STAGES);

  const long long k_begin = (long long)blockIdx.z * p.chunks_per_split * TC_KC;
  long long k_end = k_begin + (long long)p.chunks_per_split * TC_KC;
  if (k_end > p.K) k_end = p.K;
  if (k_begin >= k_end) return;  // uniform for the CTA
  const int nchunks = (int)((k_end - k_begin + TC_KC - 1) / TC_KC);

  if (warp == 0) tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // rows of this tile: m = mtile*128 + r  ->  (g, d) = (m / D, m % D); rows beyond Gr*D are zero padding
  const int rows_total = Gr * D;
  // Loader mapping (no divisions in the loop): thread -> k-row kr = tid / 4 of the chunk and a 64-byte quad of
  // 32 consecutive rows (A) / columns (B): quads `sub`, `sub + 4`, .. of A (one per tile) and of B.
  const int kr = tid >> 2, sub = tid & 3;
  const uint32_t kr_off = (uint32_t)(kr >> 3) * TC_LBO + (uint32_t)(kr & 7) * 16;
  const elem_t* a_src[J];   // delta row of quad `sub + 4 j` at k = 0
  size_t a_stride[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int m = (mtile * J + j) * TC_M + sub * 32;
    a_src[j] = nullptr; a_stride[j] = 0;
    if (m < rows_total) {
      const int g = m / D, d = m - g * D;
      if (p.cell == CELL_GRU && g == 0) { a_src[j] = p.dg0 + (size_t)n * D + d; a_stride[j] = ND; }
      else {
        const int gw = (p.cell == CELL_GRU) ? g - 1 : g;
        a_src[j] = p.dWx + (size_t)gw * ND + (size_t)n * D + d; a_stride[j] = (size_t)p.Gw * ND;
      }
    }
  }
  const int nquads = D / 32;
  // time index of this thread's k-row in the current chunk, kept incrementally (h_{t-1} of t = 0 is the initial state)
  long long kk = k_begin + kr;           // k of this thread's row in chunk 0
  long long bb = kk / T;
  int tt = (int)(kk - bb * T);
  const size_t esz = F32 ? 4 : 2;
  auto load_chunk = [&](int stage) {  // loads the NEXT chunk in sequence (chunks are requested in order)
    unsigned char* abase = smem + (size_t)stage * stage_bytes;
    unsigned char* bbase = abase + a_bytes;
    const bool krow = kk < k_end;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      unsigned char* dst = abase + (size_t)((j * 4 + sub) * 4) * TC_SBO + kr_off;
      if (krow && a_src[j] != nullptr) {
        const elem_t* src = a_src[j] + (size_t)kk * a_stride[j];
#pragma unroll
        for (int q = 0; q < 4; ++q) cp_async16(dst + (size_t)q * TC_SBO, src + q * 8);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + (size_t)q * TC_SBO) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    const unsigned char* hrow = (tt > 0)
        ? static_cast<const unsigned char*>(p.states) + ((size_t)(kk - 1) * ND + (size_t)n * D) * esz
        : static_cast<const unsigned char*>(p.s0) + ((size_t)bb * ND + (size_t)n * D) * esz;
    for (int quad = sub; quad < nquads; quad += 4) {
      unsigned char* dst = bbase + (size_t)(quad * 4) * TC_SBO + kr_off;
      if (krow) {
        if constexpr (F32) {
          const float4* src = reinterpret_cast<const float4*>(hrow) + quad * 8;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 v0 = src[2 * q], v1 = src[2 * q + 1];
            uint4 w;
            w.x = pack_x2(v0.x, v0.y); w.y = pack_x2(v0.z, v0.w);
            w.z = pack_x2(v1.x, v1.y); w.w = pack_x2(v1.z, v1.w);
            *reinterpret_cast<uint4*>(dst + (size_t)q * TC_SBO) = w;
          }
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) cp_async16(dst + (size_t)q * TC_SBO, hrow + (size_t)(quad * 4 + q) * 16);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + (size_t)q * TC_SBO) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_commit();
    kk += TC_KC;
    tt += TC_KC;
    while (tt >= T) { tt -= T; ++bb; }
  };

  const uint32_t idesc = instr_desc_16(TC_M, D, 1, 1);  // both operands MN-major
  const uint32_t smem_base = smem_u32(smem);
  bool poisoned = false;

  load_chunk(0);
  if (nchunks > 1) load_chunk(1); else cp_async_commit();
  for (int c = 0; c < nchunks; ++c) {
    const int s = c % TC_STAGES;
    if (c + 2 < nchunks) {
      const int s2 = (c + 2) % TC_STAGES;  // last read by the MMAs of chunk c-1
      if (c >= 1 && !poisoned && !mbar_wait_bounded(&bars[s2], (uint32_t)(((c - 1) / TC_STAGES) & 1))) {
        poisoned = true;
        report_timeout(p.status, c);
      }
      load_chunk(s2);
    } else {
      cp_async_commit();
    }
    cp_async_wait<2>();        // chunk c has landed (at most the two younger groups are pending)
    fence_proxy_async_smem();  // generic-proxy writes (cp.async, zero fill) -> visible to the tensor core
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t a0 = smem_base + (uint32_t)s * stage_bytes, b0 = a0 + a_bytes;
#pragma unroll
      for (int i = 0; i < TC_KC / 16; ++i) {
        const uint64_t bd = smem_desc(b0 + i * 2 * TC_LBO, TC_LBO, TC_SBO);
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const uint64_t ad = smem_desc(a0 + (uint32_t)j * (TC_M / 8) * TC_SBO + i * 2 * TC_LBO, TC_LBO, TC_SBO);
          umma_16(tmem_base + (uint32_t)(j * D), ad, bd, idesc, (c > 0 || i > 0) ? 1u : 0u);
        }
      }
      umma_commit(&bars[s]);
    }
  }
  // ---- all MMAs done -> TMEM -> global
  {
    const int last = nchunks - 1;
    if (!poisoned && !mbar_wait_bounded(&bars[last % TC_STAGES], (uint32_t)((last / TC_STAGES) & 1))) {
      poisoned = true;
      report_timeout(p.status, nchunks);
    }
  }
  tc_fence_after();
#pragma unroll 1
  for (int jt = 0; jt < J; ++jt) {
    const int m = (mtile * J + jt) * TC_M + (warp & 3) * 32 + lane;
    const bool row_ok = m < rows_total && warp < 4;
    const int g = row_ok ? m / D : 0, d = row_ok ? m - g * D : 0;
    float* out = p.dR + (((size_t)g * N + n) * D + d) * D;
    for (int col0 = 0; col0 < D; col0 += 32) {
      uint32_t r[32];
      if (warp < 4) tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(jt * D + col0), r);
      if (row_ok && !poisoned) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)  // D is a multiple of 32 here (128, 192, 256)
          red_add_f32x4(out + col0 + j, __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                        __uint_as_float(r[j + 3]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

}  // namespace

cudaError_t launch_recurrent_grad_tc(int cell, int B, int T, int N, int D, int Gr, int Gw, int state_f32, const void* dWx,
                                     const void* dg0, const void* states, const void* s0, float* dR, unsigned* status,
                                     int sm_count, cudaStream_t stream) {
  DrTcParams p;
  p.dWx = static_cast<const elem_t*>(dWx);
  p.dg0 = static_cast<const elem_t*>(dg0);
  p.states = states; p.s0 = s0; p.dR = dR; p.status = status;
  p.cell = cell; p.T = T; p.N = N; p.D = D; p.Gr = Gr; p.Gw = Gw; p.state_f32 = state_f32;
  p.K = (long long)B * T;
  const int tiles = (Gr * D + TC_M - 1) / TC_M;
  const int J = (tiles >= 2 && 2 * D <= 512) ? 2 : 1;  // two tiles per CTA where there are two to share a fetch of h
  int cols = 32;
  while (cols < J * D) cols *= 2;
  p.tmem_cols = cols;
  const int mtiles = (tiles + J - 1) / J;
  const long long chunks = (p.K + TC_KC - 1) / TC_KC;
  const long long base_ctas = (long long)mtiles * N;
  long long splits = sm_count / base_ctas;  // one CTA per SM (shared memory): stay within a single wave
  if (splits > (chunks + 3) / 4) splits = (chunks + 3) / 4;    // at least 4 chunks per split
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  p.chunks_per_split = (int)((chunks + splits - 1) / splits);
  splits = (chunks + p.chunks_per_split - 1) / p.chunks_per_split;
  const size_t smem = tc_smem_bytes(D, J);
  const dim3 grid((unsigned)mtiles, (unsigned)N, (unsigned)splits);
  auto launch = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);  // fixed: see launch_loop
    if (e != cudaSuccess) return e;
    kern<<<grid, TC_THREADS, smem, stream>>>(p);
    return cudaSuccess;
  };
  cudaError_t e;
  if (state_f32) e = J == 2 ? launch(recurrent_grad_tc_kernel<true, 2>) : launch(recurrent_grad_tc_kernel<true, 1>);
  else e = J == 2 ? launch(recurrent_grad_tc_kernel<false, 2>) : launch(recurrent_grad_tc_kernel<false, 1>);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

}  // namespace FRNN_NS
