// Shared device helpers of the sm_100a time-loop kernels: PTX wrappers (warp MMA, ldmatrix, cp.async,
// cluster barrier / distributed shared memory), fp32 gate math and the per-cell traits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "frnn_elem.cuh"

namespace FRNN_NS {

// 0..3 are the public cell ids of the C ABI.  CELL_ELMAN_CLIP is internal: Elman with forward_clip, whose backward
// needs the tanh output from before the clamp and therefore caches it (plain Elman re-reads h and caches nothing).
enum { CELL_LSTM = 0, CELL_GRU = 1, CELL_ELMAN = 2, CELL_SLSTM = 3, CELL_ELMAN_CLIP = 4 };

// Gate / state counts per cell (reference registry flashrnn/flashrnn/flashrnn.py:49-71) plus what this
// implementation caches for the backward pass and which states the backward has to re-read.
//   GC    cached values per (b,t,n,d)
//   NNEED states whose value at t-1 / t the closed-form backward needs (indices given by need(i))
//   NEXT  leading states whose external cotangent enters the backward (h, c, n; never m)
template <int CELL> struct Cell;
template <> struct Cell<CELL_LSTM> {
  static constexpr int Gr = 4, Gw = 4, Gt = 4, S = 2, GC = 4, NNEED = 1, NEXT = 2;
  __host__ __device__ static constexpr int need(int) { return 1; }
};
template <> struct Cell<CELL_GRU> {
  static constexpr int Gr = 3, Gw = 3, Gt = 4, S = 1, GC = 4, NNEED = 1, NEXT = 1;
  __host__ __device__ static constexpr int need(int) { return 0; }
};
template <> struct Cell<CELL_ELMAN> {
  static constexpr int Gr = 1, Gw = 1, Gt = 1, S = 1, GC = 0, NNEED = 1, NEXT = 1;
  __host__ __device__ static constexpr int need(int) { return 0; }
};
template <> struct Cell<CELL_ELMAN_CLIP> {
  static constexpr int Gr = 1, Gw = 1, Gt = 1, S = 1, GC = 1, NNEED = 1, NEXT = 1;
  __host__ __device__ static constexpr int need(int) { return 0; }
};
template <> struct Cell<CELL_SLSTM> {
  static constexpr int Gr = 4, Gw = 4, Gt = 4, S = 4, GC = 5, NNEED = 2, NEXT = 3;
  __host__ __device__ static constexpr int need(int i) { return i == 0 ? 1 : 2; }
};

// CELL | kNoopCell selects the measurement variant of a cell: same gate / state counts, same data movement, exchange and
// barriers, but the gate arithmetic is replaced by a pass-through.  Its step time is the floor the serial chain of the
// time loops sets without any cell math (results are meaningless).  Instantiated for the benchmark tiles only.
constexpr int kNoopCell = 8;
template <> struct Cell<CELL_LSTM | kNoopCell> : Cell<CELL_LSTM> {};
template <> struct Cell<CELL_GRU | kNoopCell> : Cell<CELL_GRU> {};
template <> struct Cell<CELL_SLSTM | kNoopCell> : Cell<CELL_SLSTM> {};

// Time steps of inputs kept in flight ahead of the step being computed (cp.async ring depth).
constexpr int kStages = 4;

// Arguments of both time-loop kernels (forward uses the first block, backward all of it).
struct LoopParams {
  const elem_t* Wx;   // [B,T,Gw,N,D]
  const uint4* Rpack;        // recurrent matrix repacked into warp-MMA A fragments
  const elem_t* bias; // [Gt,N,D]
  const void* s0;            // [S,B,1,N,D]
  void* states;              // [S,B,T,N,D]  (forward: out, backward: in)
  elem_t* cache;      // [B,T,GC,N,D] (forward: out or null, backward: in)
  const void* dstates;       // [S,B,T,N,D]
  elem_t* dWx;        // [B,T,Gw,N,D]
  elem_t* dg0;        // [B,T,N,D]   GRU only: delta of the recurrent-only gate
  void* ds0;                 // [S,B,1,N,D]
  float* dbias;              // fp32 [Gt,N,D] accumulated with atomics
  unsigned* status;
  int B, T, N, D;
  int U;                     // hidden units owned by one CTA (multiple of 16)
  int CS;                    // CTAs per cluster = D / U
  int state_f32;             // states / dstates / s0 / ds0 are fp32 (else bf16)
  float fclip, gclip;        // <= 0: off
  int grad_cut;              // backward: ignore the matrix part of the recurrent cotangent (truncated BPTT)
  int test_drop;             // test hook: CTA 0 of each cluster withholds one exchange message (see frnn_plan)
  // element strides of the caller-produced tensors (D contiguous): Wx[b][t][g][n][.], dstates[s][b][t][n][.]
  long long wx_sb, wx_st, wx_sg, wx_sn;
  long long ds_ss, ds_sb, ds_st, ds_sn;
};

// ------------------------------------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
// D(16x8, fp32) += A(16x16, elem_t, row) * B(16x8, elem_t, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32." FRNN_MMA_TYPE "." FRNN_MMA_TYPE ".f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// ---- mbarrier + bulk async copy between the shared memories of a cluster
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for a phase of `bar`, but never longer than ~1 s: on expiry the caller records the failure in
// the status block and stops waiting for the rest of the kernel (results are then invalid, the kernel ends).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > 1000000000ull) return false;
  }
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// copies `bytes` (multiple of 16) from this CTA's shared memory to the same offset space of another CTA of the
// cluster; completion is signalled as transaction bytes on the destination CTA's mbarrier
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                 uint32_t mbar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(src_cta_addr), "r"(bytes), "r"(mbar_cluster_addr) : "memory");
}
// true in exactly one lane of a fully converged warp
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred)::"memory");
  return pred != 0;
}
// Warp-collective: one elected lane of the calling (converged) warp starts the bulk copies of this CTA's slice
// [src_cta_addr, +bytes) to the same address in every other CTA of the cluster; each copy completes on the
// destination CTA's mbarrier at `bar_cta_addr`.
// Called by EVERY warp of the CTA (`warp`, `nwarps`): warp w serves the peers w, w + nwarps, ... so that the
// copies are issued in parallel.
__device__ __forceinline__ void push_slice_to_peers(uint32_t src_cta_addr, uint32_t bytes, uint32_t bar_cta_addr,
                                                    uint32_t my_rank, uint32_t cluster_size, uint32_t warp,
                                                    uint32_t nwarps) {
  __syncwarp();
#pragma unroll 1
  for (uint32_t c = warp; c < cluster_size; c += nwarps) {
    if (c == my_rank) continue;
    const uint32_t dst = map_to_cta(src_cta_addr, c), bar = map_to_cta(bar_cta_addr, c);
    if (elect_one_sync()) bulk_copy_to_cta(dst, src_cta_addr, bytes, bar);
  }
}
__device__ __forceinline__ void report_timeout(unsigned* status, int where) {
  if (atomicCAS(status, 0u, 1u) == 0u) {
    status[1] = (unsigned)where;
    status[2] = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  }
}

// four consecutive fp32 values added to global memory in one reduction (16-byte aligned address)
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ------------------------------------------------------------------------------------------------ math
// Gate nonlinearities.  Default: the hardware tanh (one MUFU op, max error ~5e-4, an order of magnitude
// below the bf16 rounding of the stored results); sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5.
// -DFRNN_EXACT_ACT switches to exp-based forms accurate to ~1e-6.
__device__ __forceinline__ float fast_tanh(float x) {
#ifndef FRNN_EXACT_ACT
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
#else
  return __fdividef(2.f, 1.f + __expf(-2.f * x)) - 1.f;
#endif
}
__device__ __forceinline__ float fast_sigmoid(float x) {
#ifndef FRNN_EXACT_ACT
  return fmaf(0.5f, fast_tanh(0.5f * x), 0.5f);
#else
  return __fdividef(1.f, 1.f + __expf(-x));
#endif
}
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - __logf(1.f + __expf(-fabsf(x))); }
__device__ __forceinline__ float clampf(float x, float v) { return fminf(fmaxf(x, -v), v); }

__device__ __forceinline__ uint32_t pack_x2(float lo, float hi) {
  elem2_t v = floats_to_elem2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_x2(uint32_t w) {
  elem2_t v = *reinterpret_cast<elem2_t*>(&w);
  return elem2_to_floats(v);
}

// Loads / stores of a pair of adjacent state values in the run-time state dtype.
__device__ __forceinline__ float2 load_state2(const void* base, size_t elem_off, int f32) {
  if (f32) return *reinterpret_cast<const float2*>(static_cast<const float*>(base) + elem_off);
  return unpack_x2(*reinterpret_cast<const uint32_t*>(static_cast<const elem_t*>(base) + elem_off));
}
__device__ __forceinline__ void store_state2(void* base, size_t elem_off, int f32, float lo, float hi) {
  if (f32) *reinterpret_cast<float2*>(static_cast<float*>(base) + elem_off) = make_float2(lo, hi);
  else *reinterpret_cast<uint32_t*>(static_cast<elem_t*>(base) + elem_off) = pack_x2(lo, hi);
}

// ------------------------------------------------------------------------------------------------ warp MMA
// acc[nt][.] (16 rows x 8*NT batch columns, fp32) = Areg (16 x 16*KT, fragments in registers) times the
// operand tile held in shared memory as `opnd[batch row][k]` (k contiguous, `stride` elements per row),
// columns kofs .. kofs+16*KT.  Independent accumulator sets keep the dependent-MMA chains short.
//
// The operand is stored as one slice per producing CTA: slice c holds, for every batch row, the `1 << ushift`
// * 16 k-columns that CTA c produces: element (b, k) sits at  (k16 >> ushift) * slice_elems + b * stride +
// kofs + (k & (16 << ushift) - 1)  where k16 = k / 16.
template <int KT, int NT>
__device__ __forceinline__ void warp_mma_rows(const uint4 (&Areg)[KT], const elem_t* opnd, int stride, int kofs,
                                              int ushift, int slice_elems, int lane, float (&out)[NT][4]) {
  // independent accumulator sets: 4 chains, 8 for the longest rows (16 k-steps: C2 forward loop 0.780 -> 0.764 ms; with
  // 8 or 12 k-steps the extra additions cost more than the shorter chains save)
  constexpr int NSETS = (KT >= 16) ? 8 : 4;
  constexpr int NACC = (NT >= NSETS) ? 1 : (NSETS / NT);
  float acc[NACC][NT][4];
#pragma unroll
  for (int a = 0; a < NACC; ++a)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][nt][c] = 0.f;
  const int j = lane >> 3, r = lane & 7;
  if constexpr (NT == 1) {
    // one ldmatrix.x4 covers two k-steps of the single 8-row batch tile
    const uint32_t base = smem_u32(opnd + r * stride + kofs + (j & 1) * 8);
    const int kmask = (1 << ushift) - 1;
#pragma unroll
    for (int k = 0; k < KT; k += 2) {
      uint32_t b0, b1, b2, b3;
      const int kk = k + (j >> 1);
      ldmatrix_x4(base + (uint32_t)(((kk >> ushift) * slice_elems + (kk & kmask) * 16) * 2), b0, b1, b2, b3);
      mma_16816(acc[k % NACC][0], Areg[k], b0, b1);
      if (k + 1 < KT) mma_16816(acc[(k + 1) % NACC][0], Areg[k + 1], b2, b3);  // odd KT: second half unused
    }
  } else {
    // one ldmatrix.x4 covers one k-step of two 8-row batch tiles
    const uint32_t base = smem_u32(opnd + ((j >> 1) * 8 + r) * stride + kofs + (j & 1) * 8);
    const int kmask = (1 << ushift) - 1;
#pragma unroll
    for (int k = 0; k < KT; ++k) {
      const uint32_t koff = (uint32_t)(((k >> ushift) * slice_elems + (k & kmask) * 16) * 2);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(base + koff + (uint32_t)(np * 16 * stride * 2), b0, b1, b2, b3);
        mma_16816(acc[k % NACC][2 * np], Areg[k], b0, b1);
        mma_16816(acc[k % NACC][2 * np + 1], Areg[k], b2, b3);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float s = acc[0][nt][c];
#pragma unroll
      for (int a = 1; a < NACC; ++a) s += acc[a][nt][c];
      out[nt][c] = s;
    }
}

// Continues such a product over the k-steps [k0, k1) whose A fragments do not fit the register file and are streamed
// from global memory every time step (head dims above 256): fragment k of this warp's row tile sits at asrc[k * 32]
// (lane offset already applied).  Accumulates into `acc`.  k1 - k0 must be even.
// SMEM: the fragments are a copy of that range kept in shared memory (plain loads) instead of global memory.
template <int NT, bool SMEM = false>
__device__ __forceinline__ void warp_mma_stream(const uint4* asrc, int k0, int k1, const elem_t* opnd, int stride,
                                                int kofs, int ushift, int slice_elems, int lane, float (&acc)[NT][4]) {
  auto frag = [&](int k) -> uint4 {
    if constexpr (SMEM) return asrc[(size_t)k * 32];
    else return __ldg(asrc + (size_t)k * 32);
  };
  const int j = lane >> 3, r = lane & 7;
  const int kmask = (1 << ushift) - 1;
  // (one accumulator chain: four independent chains were measured and lost -- head dim 768 forward loop 3.64 -> 3.89 ms,
  // reverse loop 5.00 -> 6.47 ms)
  if constexpr (NT == 1) {
    const uint32_t base = smem_u32(opnd + r * stride + kofs + (j & 1) * 8);
#pragma unroll 2
    for (int k = k0; k < k1; k += 2) {
      const uint4 a0 = frag(k), a1 = frag(k + 1);
      uint32_t b0, b1, b2, b3;
      const int kk = k + (j >> 1);
      ldmatrix_x4(base + (uint32_t)(((kk >> ushift) * slice_elems + (kk & kmask) * 16) * 2), b0, b1, b2, b3);
      mma_16816(acc[0], a0, b0, b1);
      mma_16816(acc[0], a1, b2, b3);
    }
  } else {
    const uint32_t base = smem_u32(opnd + ((j >> 1) * 8 + r) * stride + kofs + (j & 1) * 8);
#pragma unroll 2
    for (int k = k0; k < k1; ++k) {
      const uint4 a = frag(k);
      const uint32_t koff = (uint32_t)(((k >> ushift) * slice_elems + (k & kmask) * 16) * 2);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(base + koff + (uint32_t)(np * 16 * stride * 2), b0, b1, b2, b3);
        mma_16816(acc[2 * np], a, b0, b1);
        mma_16816(acc[2 * np + 1], a, b2, b3);
      }
    }
  }
}

// Same product for MT row tiles that share the operand: out[m] = A_m (16 x 16*KP, fragments Areg[m*KP + k]) times the
// contiguous tile `opnd[batch row][k]`.  The operand fragments are loaded once per k-step and reused by all MT tiles.
template <int MT, int KP, int NT>
__device__ __forceinline__ void warp_mma_tiles(const uint4* Areg, const elem_t* opnd, int stride, int lane,
                                               float (&out)[MT][NT][4]) {
  constexpr int NACC = (MT * NT >= 4) ? 1 : (4 / (MT * NT));
  float acc[NACC][MT][NT][4];
#pragma unroll
  for (int a = 0; a < NACC; ++a)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][m][nt][c] = 0.f;
  const int j = lane >> 3, r = lane & 7;
  if constexpr (NT == 1) {
    const uint32_t base = smem_u32(opnd + r * stride + (j >> 1) * 16 + (j & 1) * 8);
#pragma unroll
    for (int k = 0; k < KP; k += 2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(base + (uint32_t)(k * 32), b0, b1, b2, b3);  // k-steps k and k+1 (the latter unused when KP is odd)
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        mma_16816(acc[k % NACC][m][0], Areg[m * KP + k], b0, b1);
        if (k + 1 < KP) mma_16816(acc[(k + 1) % NACC][m][0], Areg[m * KP + k + 1], b2, b3);
      }
    }
  } else {
    const uint32_t base = smem_u32(opnd + ((j >> 1) * 8 + r) * stride + (j & 1) * 8);
#pragma unroll
    for (int k = 0; k < KP; ++k) {
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(base + (uint32_t)((np * 16 * stride + k * 16) * 2), b0, b1, b2, b3);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          mma_16816(acc[k % NACC][m][2 * np], Areg[m * KP + k], b0, b1);
          mma_16816(acc[k % NACC][m][2 * np + 1], Areg[m * KP + k], b2, b3);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float s = acc[0][m][nt][c];
#pragma unroll
        for (int a = 1; a < NACC; ++a) s += acc[a][m][nt][c];
        out[m][nt][c] = s;
      }
}

// Threads per CTA the kernels are compiled for, by k-steps held in registers per warp.
// Slot rows of the per-thread prefetch rings: threads beyond the item count of the CTA own no items and no slots
// (8-row batch tiles of the 4-gate cells keep only every second thread busy in the pointwise phase).
__host__ __device__ constexpr int ring_row_len(int U, int BT, int threads) {
  return (U / 2) * BT < threads ? (U / 2) * BT : threads;
}

// Streamed kernels (head dims above 256): of the k-steps of R that do not fit a warp's registers, as many as the rest of
// the shared-memory budget holds stay there for all T steps (one 512-byte fragment set per warp and k-step, an even
// number of them); only what is left is re-read from L2 in every step.  `base_bytes` = the kernel's other shared memory.
constexpr int kStreamKT = 8;      // k-steps of R a warp of the streamed kernels keeps in registers
constexpr int kStreamU = 64;      // units per CTA of the streamed kernels (cluster size D / 64, up to 16)
constexpr int kStreamMaxD = 1024;
constexpr size_t kSmemBudget = 227 * 1024;
__host__ __device__ constexpr int stream_ksm(int D, int kt_regs, int threads, size_t base_bytes) {
  const int want = D / 16 - kt_regs;
  const size_t per = (size_t)(threads / 32) * 512;
  if (want <= 0 || base_bytes + 64 >= kSmemBudget) return 0;
  const int fit = (int)((kSmemBudget - base_bytes - 64) / per) & ~1;
  return fit < want ? fit : want;
}

template <int KT> struct MaxThreads { static constexpr int v = (KT >= 16) ? 256 : (KT >= 12) ? 384 : 512; };
// Launch bounds per (cell, KT): a CTA never has more than 2*Gr*D threads (U <= D).  No minimum-blocks hint: capping
// the registers of the small-head kernels to raise occupancy (6 instead of 4 CTAs per SM) made the Elman D=64
// backward 70 % slower on B200 (measured), so the compiler is left free.
template <int CELL, int KT> struct LaunchBounds {
  static constexpr int cap = MaxThreads<KT>::v;
  static constexpr int full = 32 * Cell<CELL>::Gr * KT;
  static constexpr int threads = full < cap ? full : cap;
  static constexpr int min_blocks = 1;
};

}  // namespace FRNN_NS
