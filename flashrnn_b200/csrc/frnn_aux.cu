// Helper kernels around the time loops:
//   pack_recurrent_kernel  R[Gr,N,D,D] -> warp-MMA A fragments (forward: R, backward: R^T)
//   recurrent_grad_kernel  dR[g,n,d,p] = sum_{b,t} delta_g[b,t,n,d] * h_{t-1}[b,n,p]   (split-K tensor-core GEMM)
//   cast_grads_kernel      fp32 dR || db -> parameter dtype
#include "frnn_aux.cuh"

namespace FRNN_NS {

// One thread builds one 16-byte fragment (what one lane holds of one 16x16 A tile of mma.m16n8k16):
//   out[((n*Gr + g)*(D/16) + ut)*(D/16) + k][lane] ;  A[row][kk], row/kk in 0..15
//   forward : A[row][kk] = R[g][n][ut*16 + row][k*16 + kk]
//   backward: A[row][kk] = R[g][n][k*16 + kk][ut*16 + row]      (rows = input unit p)
__global__ void pack_recurrent_kernel(const elem_t* __restrict__ R, uint4* __restrict__ out, int Gr, int N, int D,
                                      int transpose) {
  const int KT = D / 16;
  const size_t total = (size_t)N * Gr * KT * KT * 32;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int lane = (int)(idx & 31);
  size_t r = idx >> 5;
  const int k = (int)(r % KT); r /= KT;
  const int ut = (int)(r % KT); r /= KT;
  const int g = (int)(r % Gr);
  const int n = (int)(r / Gr);
  const int gid = lane >> 2, tig = lane & 3;
  const elem_t* Rg = R + (((size_t)g * N + n) * D) * D;
  auto at = [&](int row, int kk) -> unsigned short {
    const int a = ut * 16 + row, c = k * 16 + kk;
    const elem_t v = transpose ? Rg[(size_t)c * D + a] : Rg[(size_t)a * D + c];
    return *reinterpret_cast<const unsigned short*>(&v);
  };
  auto pair = [&](int row, int kk) -> uint32_t { return (uint32_t)at(row, kk) | ((uint32_t)at(row, kk + 1) << 16); };
  uint4 v;
  v.x = pair(gid, 2 * tig);
  v.y = pair(gid + 8, 2 * tig);
  v.z = pair(gid, 2 * tig + 8);
  v.w = pair(gid + 8, 2 * tig + 8);
  out[idx] = v;
}

// ---------------------------------------------------------------------------------------------------------
// dR.  For one R gate g and head n:  C[d][p] = sum_k A_k[d] * H_k[p],  k = b*T + t,
//   A_k = delta of gate g at (b,t) (a row of dWx, or of the GRU side buffer), H_k = h_{t-1}[b] (a row of
//   states[0] shifted by one step; the initial h for t == 0).
// CTA tile 64(d) x 64(p), 4 warps (2x2, 32x32 each), K chunks of 32 double-buffered with cp.async; both
// operands sit in shared memory k-major and are transposed on the fly by ldmatrix.trans.  Split-K over
// gridDim.z with fp32 atomics into the gradient workspace.
constexpr int DR_TM = 64, DR_TN = 64, DR_KC = 32, DR_LD = 72;  // 72*2 B = 144 B row pitch: conflict-free ldmatrix

struct DrParams {
  const elem_t* dWx;  // [B,T,Gw,N,D]
  const elem_t* dg0;  // [B,T,N,D] (GRU)
  const void* states;        // [S,B,T,N,D]; only s = 0 is read
  const void* s0;            // [S,B,1,N,D]
  float* dR;                 // [Gr,N,D,D] fp32
  int cell, B, T, N, D, Gr, Gw, state_f32;
  long long K;               // B*T
  int chunks_per_split;
};

template <bool F32>
__global__ void __launch_bounds__(128) recurrent_grad_kernel(const DrParams p) {
  __shared__ __align__(16) elem_t As[2][DR_KC][DR_LD];
  __shared__ __align__(16) elem_t Hs[2][DR_KC][DR_LD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = p.D, N = p.N, T = p.T;
  const int tiles = (D + DR_TM - 1) / DR_TM;
  const int tm = blockIdx.x / tiles, tn = blockIdx.x % tiles;
  const int g = blockIdx.y / N, n = blockIdx.y % N;
  const size_t ND = (size_t)N * D;

  // source of the delta rows of R-gate g
  const elem_t* abase;
  size_t astride;
  if (p.cell == CELL_GRU) {
    if (g == 0) { abase = p.dg0 + (size_t)n * D; astride = ND; }
    else { abase = p.dWx + (size_t)(g - 1) * ND + (size_t)n * D; astride = (size_t)p.Gw * ND; }
  } else {
    abase = p.dWx + (size_t)g * ND + (size_t)n * D;
    astride = (size_t)p.Gw * ND;
  }
  const long long k_begin = (long long)blockIdx.z * p.chunks_per_split * DR_KC;
  long long k_end = k_begin + (long long)p.chunks_per_split * DR_KC;
  if (k_end > p.K) k_end = p.K;
  if (k_begin >= k_end) return;
  const int nchunks = (int)((k_end - k_begin + DR_KC - 1) / DR_KC);

  // each thread moves 2 x 16 B of each operand per chunk: rows r0 and r0+16, 8 columns at c8
  const int r0 = tid >> 3, c8 = (tid & 7) * 8;
  auto load_chunk = [&](int chunk, int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = r0 + h * 16;
      const long long k = k_begin + (long long)chunk * DR_KC + r;
      const bool krow = k < k_end;
      // delta rows
      {
        const int d = tm * DR_TM + c8;
        elem_t* dst = &As[buf][r][c8];
        if (krow && d < D) cp_async16(dst, abase + (size_t)k * astride + d);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
      }
      // h_{t-1} rows
      {
        const int pcol = tn * DR_TN + c8;
        elem_t* dst = &Hs[buf][r][c8];
        if (krow && pcol < D) {
          const long long b = k / T;
          const int t = (int)(k - b * T);
          const size_t off = (t > 0) ? ((size_t)(k - 1)) * ND + (size_t)n * D + pcol
                                     : ((size_t)b) * ND + (size_t)n * D + pcol;
          const void* base = (t > 0) ? p.states : p.s0;
          if constexpr (F32) {
            const float4 v0 = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
            const float4 v1 = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + off + 4);
            uint4 w;
            w.x = pack_x2(v0.x, v0.y); w.y = pack_x2(v0.z, v0.w);
            w.z = pack_x2(v1.x, v1.y); w.w = pack_x2(v1.z, v1.w);
            *reinterpret_cast<uint4*>(dst) = w;
          } else {
            cp_async16(dst, static_cast<const elem_t*>(base) + off);
          }
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    cp_async_commit();
  };

  float acc[2][4][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const int j = lane >> 3, r = lane & 7;
  load_chunk(0, 0);
  for (int c = 0; c < nchunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < nchunks) { load_chunk(c + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < DR_KC / 16; ++ks) {
      uint4 afr[2];
      uint32_t bfr[4][2];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)  // A(m,k) = As[k][m]: matrices (k lo, m lo), (k lo, m hi), (k hi, m lo), (k hi, m hi)
        ldmatrix_x4_trans(smem_u32(&As[buf][ks * 16 + (j >> 1) * 8 + r][wm + mt * 16 + (j & 1) * 8]), afr[mt].x,
                          afr[mt].y, afr[mt].z, afr[mt].w);
#pragma unroll
      for (int np = 0; np < 2; ++np)  // B(k,n) = Hs[k][n]: matrices (k lo, n0), (k hi, n0), (k lo, n1), (k hi, n1)
        ldmatrix_x4_trans(smem_u32(&Hs[buf][ks * 16 + (j & 1) * 8 + r][wn + np * 16 + (j >> 1) * 8]), bfr[2 * np][0],
                          bfr[2 * np][1], bfr[2 * np + 1][0], bfr[2 * np + 1][1]);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma_16816(acc[mt][nt], afr[mt], bfr[nt][0], bfr[nt][1]);
    }
    __syncthreads();
  }

  const int gid = lane >> 2, tig = lane & 3;
  float* out = p.dR + (((size_t)g * N + n) * D) * D;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int d = tm * DR_TM + wm + mt * 16 + gid + (c >> 1) * 8;
        const int pc = tn * DR_TN + wn + nt * 8 + 2 * tig + (c & 1);
        if (d < D && pc < D) atomicAdd(out + (size_t)d * D + pc, acc[mt][nt][c]);
      }
}

__global__ void cast_grads_kernel(const float* __restrict__ src, elem_t* __restrict__ dR, elem_t* __restrict__ db,
                                  size_t nR, size_t nb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nR) dR[i] = float_to_elem(src[i]);
  else if (i < nR + nb) db[i - nR] = float_to_elem(src[i]);
}

// ---------------------------------------------------------------------------------------------------------
cudaError_t launch_pack_recurrent(const void* R, void* out, int Gr, int N, int D, int transpose, cudaStream_t stream) {
  const int KT = D / 16;
  const size_t total = (size_t)N * Gr * KT * KT * 32;
  const int threads = 256;
  pack_recurrent_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
      static_cast<const elem_t*>(R), static_cast<uint4*>(out), Gr, N, D, transpose);
  return cudaGetLastError();
}

cudaError_t launch_recurrent_grad(int cell, int B, int T, int N, int D, int Gr, int Gw, int state_f32, const void* dWx,
                                  const void* dg0, const void* states, const void* s0, float* dR, int sm_count,
                                  cudaStream_t stream) {
  DrParams p;
  p.dWx = static_cast<const elem_t*>(dWx);
  p.dg0 = static_cast<const elem_t*>(dg0);
  p.states = states; p.s0 = s0; p.dR = dR;
  p.cell = cell; p.B = B; p.T = T; p.N = N; p.D = D; p.Gr = Gr; p.Gw = Gw; p.state_f32 = state_f32;
  p.K = (long long)B * T;
  const int tiles = (D + DR_TM - 1) / DR_TM;
  const long long chunks = (p.K + DR_KC - 1) / DR_KC;
  const long long base_ctas = (long long)tiles * tiles * Gr * N;
  // aim for ~4 waves of CTAs; every split handles at least 8 chunks so the atomics stay a small share
  long long splits = (4LL * sm_count + base_ctas - 1) / base_ctas;
  if (splits > (chunks + 7) / 8) splits = (chunks + 7) / 8;
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  p.chunks_per_split = (int)((chunks + splits - 1) / splits);
  splits = (chunks + p.chunks_per_split - 1) / p.chunks_per_split;
  dim3 grid((unsigned)(tiles * tiles), (unsigned)(Gr * N), (unsigned)splits);
  if (state_f32) recurrent_grad_kernel<true><<<grid, 128, 0, stream>>>(p);
  else recurrent_grad_kernel<false><<<grid, 128, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_cast_grads(const float* src, void* dR, void* db, size_t nR, size_t nb, cudaStream_t stream) {
  const size_t total = nR + nb;
  const int threads = 256;
  cast_grads_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
      src, static_cast<elem_t*>(dR), static_cast<elem_t*>(db), nR, nb);
  return cudaGetLastError();
}

}  // namespace FRNN_NS
