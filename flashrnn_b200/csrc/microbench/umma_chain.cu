// Microbenchmark behind one entry of the tile table: should the per-step gate product of the small-batch time loops
// (one CTA: 128 gate rows x K = 256, 8-16 batch columns) run on the 5th-generation tensor cores?
// It times that product as a tcgen05 chain per time step -- A operand (the CTA's 128 x 256 slice of R) resident in
// TENSOR MEMORY, or in shared memory for comparison; B = the h tile [16 batch rows][K = 256] in shared memory; a 16-column
// accumulator -- with everything a step of the recurrence needs around it: the h tile is touched and fenced for the
// tensor cores, a CTA barrier, one thread issues the 16 MMAs (K = 16 each) and a commit, all threads wait on the
// mbarrier and read their accumulator row with tcgen05.ld.  The result is checked against a host product.
// The warp-MMA phase it competes with (R in registers, mma.sync, pre-activations through shared memory) takes
// ~360 clk + a ~100 clk barrier in the forward loop of the same tile.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I flashrnn_b200/csrc -o umma_chain flashrnn_b200/csrc/microbench/umma_chain.cu && ./umma_chain
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cmath>
#include "frnn_tc.cuh"

using namespace frnn;

constexpr int M = 128, K = 256, NB = 16, KS = K / 16;

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem)
__device__ __forceinline__ void umma_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// R: [M][K] bf16 row-major (global); h: [NB][K] bf16; out: [M][NB] fp32 of the LAST step's product; clk: phase sums
template <bool A_TMEM>
__global__ void __launch_bounds__(128, 1) probe(const __nv_bfloat16* R, const __nv_bfloat16* h, float* out, long long* clk,
                                                unsigned* status, int steps) {
  extern __shared__ __align__(1024) unsigned char smem[];
  // B tile: [n/8][k/8][8][16 B]  (LBO = 128 between k groups, SBO = 4096 between n groups): 8 KB
  unsigned char* btile = smem;
  unsigned char* atile = smem + 8192;                        // A_TMEM == false: [m/8][k/8][8][16 B], 64 KB
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 8192 + 65536);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  if (tid == 0) { mbar_init(bar, 1); fence_mbar_init(); }
  // h tile
  for (int i = tid; i < NB * K / 8; i += 128) {
    const int n = i / (K / 8), kg = i % (K / 8);
    *reinterpret_cast<uint4*>(btile + (n / 8) * 4096 + kg * 128 + (n % 8) * 16) = *reinterpret_cast<const uint4*>(h + n * K + kg * 8);
  }
  if (!A_TMEM)
    for (int i = tid; i < M * K / 8; i += 128) {
      const int m = i / (K / 8), kg = i % (K / 8);
      *reinterpret_cast<uint4*>(atile + (m / 8) * 4096 + kg * 128 + (m % 8) * 16) = *reinterpret_cast<const uint4*>(R + m * K + kg * 8);
    }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_a = tmem, tmem_d = tmem + 128;        // A: columns 0..127 (K = 256 bf16), D: columns 128..143
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  if (A_TMEM) {  // row m = tid: 256 bf16 = 128 columns, 8 columns (one k-step) per store
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t r[8];
      const uint4 a = *reinterpret_cast<const uint4*>(R + tid * K + ks * 16), b = *reinterpret_cast<const uint4*>(R + tid * K + ks * 16 + 8);
      r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w; r[4] = b.x; r[5] = b.y; r[6] = b.z; r[7] = b.w;
      tmem_st8(tmem_a + lane_base + ks * 8, r);
    }
    tmem_st_wait();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t idesc = instr_desc_16(M, NB, 0, 0);
  long long sum[4] = {0, 0, 0, 0}, last = clock64();
  float keep = 0.f;
  bool ok = true;
  uint32_t d[16];
  for (int t = 0; t < steps && ok; ++t) {
    // (0) stand-in for "h_t written by the cell phase": every thread rewrites 16 bytes of the tile, then the proxy fence
    {
      uint4* p = reinterpret_cast<uint4*>(btile + (tid / 64) * 4096 + (tid % 32) * 128 + ((tid / 32) % 2 * 4) * 16);
      uint4 v = *p; v.x ^= 0u; *p = v;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    { const long long c = clock64(); sum[0] += c - last; last = c; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t b0 = smem_u32(btile);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const uint64_t bd = smem_desc(b0 + ks * 256, 128, 4096);
        if (A_TMEM) umma_ta(tmem_d, tmem_a + ks * 8, bd, idesc, ks > 0);
        else umma_16(tmem_d, smem_desc(smem_u32(atile) + ks * 256, 128, 4096), bd, idesc, ks > 0);
      }
      umma_commit(bar);
    }
    { const long long c = clock64(); sum[1] += c - last; last = c; }
    if (!mbar_wait_bounded(bar, (uint32_t)(t & 1))) { ok = false; atomicExch(status, 1u + t); }
    tc_fence_after();
    { const long long c = clock64(); sum[2] += c - last; last = c; }
    tmem_ld16(tmem_d + lane_base, d);
    keep += __uint_as_float(d[t & 15]);
    { const long long c = clock64(); sum[3] += c - last; last = c; }
  }
  if (ok)
    for (int j = 0; j < 16; ++j) out[tid * NB + j] = __uint_as_float(d[j]);
  if (tid == 0 || tid == 64) for (int i = 0; i < 4; ++i) clk[(tid ? 4 : 0) + i] = sum[i];
  if (keep == 123.456f) out[0] = keep;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

int main() {
  std::vector<__nv_bfloat16> R(M * K), h(NB * K);
  std::vector<float> Rf(M * K), hf(NB * K);
  srand(1);
  for (int i = 0; i < M * K; ++i) { float v = (rand() % 2001 - 1000) / 16000.f; R[i] = __float2bfloat16(v); Rf[i] = __bfloat162float(R[i]); }
  for (int i = 0; i < NB * K; ++i) { float v = (rand() % 2001 - 1000) / 1000.f; h[i] = __float2bfloat16(v); hf[i] = __bfloat162float(h[i]); }
  __nv_bfloat16 *dR, *dh; float* dout; long long* dclk; unsigned* dst;
  cudaMalloc(&dR, M * K * 2); cudaMalloc(&dh, NB * K * 2); cudaMalloc(&dout, M * NB * 4); cudaMalloc(&dclk, 64); cudaMalloc(&dst, 4);
  cudaMemcpy(dR, R.data(), M * K * 2, cudaMemcpyHostToDevice); cudaMemcpy(dh, h.data(), NB * K * 2, cudaMemcpyHostToDevice);
  const int smem = 8192 + 65536 + 64;
  const int steps = 2000;
  for (int variant = 0; variant < 2; ++variant) {
    auto kern = variant == 0 ? probe<true> : probe<false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaMemset(dst, 0, 4); cudaMemset(dout, 0, M * NB * 4);
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    kern<<<1, 128, smem>>>(dR, dh, dout, dclk, dst, 10);
    cudaEventRecord(e0);
    kern<<<1, 128, smem>>>(dR, dh, dout, dclk, dst, steps);
    cudaEventRecord(e1);
    cudaError_t e = cudaDeviceSynchronize();
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    std::vector<float> out(M * NB); long long clk[8]; unsigned st;
    cudaMemcpy(out.data(), dout, M * NB * 4, cudaMemcpyDeviceToHost); cudaMemcpy(clk, dclk, 64, cudaMemcpyDeviceToHost); cudaMemcpy(&st, dst, 4, cudaMemcpyDeviceToHost);
    double maxerr = 0;
    for (int m = 0; m < M; ++m) for (int n = 0; n < NB; ++n) {
      double ref = 0; for (int k = 0; k < K; ++k) ref += (double)Rf[m * K + k] * hf[n * K + k];
      maxerr = fmax(maxerr, fabs(ref - out[m * NB + n]));
    }
    printf("variant %s: cuda=%s status=%u  %.1f ns/step  max|err|=%.3e\n", variant == 0 ? "A in TMEM" : "A in smem", cudaGetErrorString(e), st,
           ms * 1e6 / steps, maxerr);
    for (int who = 0; who < 2; ++who)
      printf("  thread %3d clk/step: write+fence+barrier %.0f | issue 16 MMA + commit %.0f | wait mbarrier %.0f | tcgen05.ld %.0f\n", who * 64,
             clk[who * 4 + 0] / (double)steps, clk[who * 4 + 1] / (double)steps, clk[who * 4 + 2] / (double)steps, clk[who * 4 + 3] / (double)steps);
  }
  return 0;
}
