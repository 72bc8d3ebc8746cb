// C ABI of libfrnn_b200.so (declared in include/frnn.h): validation, tile selection, launches.
// No device memory is allocated or freed here and the host is never synchronised with the device,
// except in frnn_read_device_status.
#include "../../include/frnn.h"

#include <mutex>

#include "frnn_aux.cuh"

namespace FRNN_NS {

struct CellDims { int Gr, Gw, Gt, S, GC; };
static bool cell_dims(int cell, CellDims* d) {
  switch (cell) {
    case CELL_LSTM:  *d = {4, 4, 4, 2, 4}; return true;
    case CELL_GRU:   *d = {3, 3, 4, 1, 4}; return true;
    case CELL_ELMAN: *d = {1, 1, 1, 1, 1}; return true;
    case CELL_SLSTM: *d = {4, 4, 4, 4, 5}; return true;
  }
  return false;
}

LoopKernel get_fwd_kernel(int cell, int kt, int nt) {
  switch (cell) {
    case CELL_LSTM: return get_fwd_kernel_lstm(kt, nt);
    case CELL_GRU: return get_fwd_kernel_gru(kt, nt);
    case CELL_ELMAN: return get_fwd_kernel_elman(kt, nt);
    case CELL_ELMAN_CLIP: return get_fwd_kernel_elmanc(kt, nt);
    case CELL_SLSTM: return get_fwd_kernel_slstm(kt, nt);
  }
  return LoopKernel{nullptr, 0, nullptr};
}
LoopKernel get_bwd_kernel(int cell, int kt, int nt, int mpw) {
  switch (cell) {
    case CELL_LSTM: return get_bwd_kernel_lstm(kt, nt, mpw);
    case CELL_GRU: return get_bwd_kernel_gru(kt, nt, mpw);
    case CELL_ELMAN: return get_bwd_kernel_elman(kt, nt, mpw);
    case CELL_ELMAN_CLIP: return get_bwd_kernel_elmanc(kt, nt, mpw);
    case CELL_SLSTM: return get_bwd_kernel_slstm(kt, nt, mpw);
  }
  return LoopKernel{nullptr, 0, nullptr};
}

// kernel family of a problem: the public cell id, except Elman with a forward clamp (caches its tanh output)
static int kernel_cell(const frnn_problem& pr) {
  return (pr.cell == CELL_ELMAN && pr.forward_clip > 0.f) ? (int)CELL_ELMAN_CLIP : pr.cell;
}

// Activation values cached per (b,t,n,d) in training.  Elman needs its one slot (the tanh output) only when h is
// clamped afterwards; otherwise h itself serves and no cache buffer is needed at all.
static int cache_slots_of(const frnn_problem& pr, const CellDims& cd) {
  return (pr.cell == CELL_ELMAN && !(pr.forward_clip > 0.f)) ? 0 : cd.GC;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
constexpr size_t kMaxDynSmem = 227 * 1024;
constexpr size_t kStatusBytes = 256;

struct WsLayout { size_t rpack_fwd, rpack_bwd, grads, dg0, total; };
static WsLayout workspace_layout(const frnn_problem& pr, const CellDims& cd) {
  WsLayout w;
  const size_t rbytes = (size_t)cd.Gr * pr.N * pr.D * pr.D * 2;
  size_t off = kStatusBytes;
  w.rpack_fwd = off; off = align_up(off + rbytes, 256);
  w.rpack_bwd = off; off = align_up(off + rbytes, 256);
  w.grads = off; off = align_up(off + ((size_t)cd.Gr * pr.N * pr.D * pr.D + (size_t)cd.Gt * pr.N * pr.D) * 4, 256);
  w.dg0 = off;
  if (pr.cell == CELL_GRU) off = align_up(off + (size_t)pr.B * pr.T * pr.N * pr.D * 2, 256);
  w.total = off;
  return w;
}

// Backward exchange scheme of a tile: reduce-scatter (returns MPW = CS / Gr) where that kernel exists and fits,
// else all-gather (0).
// head dims above 256 take the streamed kernels (lookup key kt = 0)
static bool streamed(const frnn_problem& pr) { return pr.D > 256; }
static int kernel_kt(const frnn_problem& pr) { return streamed(pr) ? 0 : pr.D / 16; }

static int bwd_mpw(const frnn_problem& pr, const CellDims& cd, int cs, int bt) {
  if (streamed(pr) || cs <= 1 || cs % cd.Gr) return 0;
  const int U = pr.D / cs, threads = 2 * cd.Gr * U, mpw = cs / cd.Gr;
  const LoopKernel k = get_bwd_kernel(kernel_cell(pr), pr.D / 16, bt / 8, mpw);
  if (!k.fn || threads > k.max_threads || k.smem_bytes(pr.D, U, threads) > kMaxDynSmem) return 0;
  return mpw;
}

// A tile (cluster size, batch tile) is usable when both loop kernels exist for it, the CTA fits the
// instantiation's thread bound and the shared-memory budget.
static bool wide_problem(const frnn_problem& pr) {
  return wide_supported(pr.cell, pr.D, pr.dtype_state == FRNN_DTYPE_F32, pr.forward_clip, pr.grad_clip, pr.grad_cut);
}
static bool is_wide(const frnn_plan& pl) { return pl.batch_tile == kWideBatchTile; }
// LSTM and GRU at head dim 64: the forward loop alone has a 128-row form (the reverse loop stays on 16-row tiles)
static bool wide_gates_problem(const frnn_problem& pr) {
  return wide_gates_forward_supported(pr.cell, pr.D, pr.dtype_state == FRNN_DTYPE_F32);
}
static int plan_threads(const CellDims& cd, int units, int bt) { return bt == kWideBatchTile ? kWideThreads : 2 * cd.Gr * units; }

static bool tile_ok(const frnn_problem& pr, const CellDims& cd, int cs, int bt) {
  const int D = pr.D;
  if (bt == kWideBatchTile) return cs == 1 && wide_problem(pr);  // 128-row tensor-core loops: one CTA per head and tile
  if (cs < 1 || D % cs) return false;
  // clusters above 8 CTAs (a non-portable size): the streamed kernels, and 16 CTAs of 16 units for head dim 256
  if (streamed(pr) ? (cs > 16 || D / cs != kStreamU) : (cs > 8 && !(cs == 16 && D == 256))) return false;
  const int U = D / cs;
  if (U % 16 || ((U / 16) & (U / 16 - 1))) return false;  // 16 * power of two
  if (bt != 8 && bt != 16 && bt != 32) return false;
  const int kt = kernel_kt(pr), nt = bt / 8, threads = 2 * cd.Gr * U;
  const LoopKernel f = get_fwd_kernel(kernel_cell(pr), kt, nt), b = get_bwd_kernel(kernel_cell(pr), kt, nt, 0);
  if (!f.fn || !b.fn) return false;
  if (threads > f.max_threads || threads > b.max_threads || threads < 32) return false;
  if (f.smem_bytes(D, U, threads) > kMaxDynSmem || b.smem_bytes(D, U, threads) > kMaxDynSmem) return false;
  return true;
}

static int sm_count_cached();

// Default tile per problem.  Small-batch problems are bound by the per-step latency of the serial chain, so
// the head is spread over as many SMs as a portable cluster allows; large-batch problems already fill the
// GPU with (head, batch tile) pairs and take the smallest cluster (no cross-CTA exchange when it is 1).
static bool choose_tile(const frnn_problem& pr, const CellDims& cd, int want_cs, int want_bt, int* cs_out, int* bt_out) {
  // Large batches of a cell / head dim the 128-row tensor-core loops cover: those stream at the HBM rate once their
  // (head, 128-row tile) pairs occupy most of the SMs
  if (want_bt == kWideBatchTile && wide_gates_problem(pr)) want_bt = 16;  // 128-row forward loop over 16-row reverse tiles
  if ((want_bt == kWideBatchTile || (!want_bt && !want_cs && (long long)(pr.B / kWideBatchTile) * pr.N >= 64)) &&
      tile_ok(pr, cd, 1, kWideBatchTile) && (want_cs == 0 || want_cs == 1)) {
    *cs_out = 1;
    *bt_out = kWideBatchTile;
    return true;
  }
  // Measured on B200.  Small batches (fewer than 128 (head, batch tile) pairs; every benchmark configuration but the large
  // Elman one): 8-row batch tiles -- more CTAs, shorter steps; 16-row tiles double the step time of the serial chain.
  // Large batches of the cells with three or four gates: 16-row tiles, whose CTAs reuse every fragment of R for two
  // 8-row MMA columns (LSTM B1024 N16 D64: 55 -> 72 M tokens/s through the two loops; GRU 64 -> 75; sLSTM 82 -> 96; LSTM
  // B512 N8 D128 37 -> 48; 32-row tiles spill in the reverse loop and lose).  Elman keeps 8 rows (D=128: 100 against 72).
  const bool rows16 = cd.Gr >= 3 && (long long)((pr.B + 15) / 16) * pr.N >= 128;
  const int bt_pref[3] = {rows16 ? 16 : 8, rows16 ? 8 : 16, 32};
  for (int bi = 0; bi < 3; ++bi) {
    const int bt = want_bt ? want_bt : bt_pref[bi];
    const long long pairs = (long long)((pr.B + bt - 1) / bt) * pr.N;
    const bool fill = pairs >= 128;
    // power-of-two cluster sizes first, then the others
    const int order_small[8] = {8, 4, 2, 1, 6, 3, 7, 5};
    const int order_large[8] = {1, 2, 4, 8, 3, 6, 5, 7};
    const int sms = sm_count_cached();
    // The preferred cluster, small batch or large: 32 units per CTA from head dim 128 (clusters of D/32), the whole head in
    // one CTA up to head dim 64.  16-unit CTAs (3-4 warps each) lose more in the exchange than they gain in the matrix
    // phase (GRU head dim 128, 16 pairs: clusters of 8 x 16 units 3.54 ms, 4 x 32 units 3.03 ms, 2 x 64 3.37 ms; LSTM head dim
    // 256: 16 x 16 units 1.07 ms per forward loop against 0.78 ms for 8 x 32; large batch LSTM D=128: 4 x 32 units 48, 2 x 64
    // units 41 M tokens/s); up to head dim 64 one CTA per head, no exchange at all, wins (LSTM D=64, 2 pairs: fwd + bwd
    // loops 0.33 ms against 0.35 / 0.36 ms for clusters of 2 / 4; Elman D=64: 0.46 against 0.65 / 0.81 ms; large batch LSTM
    // D=64: 72 against 66 M tokens/s).
    // Small batches fall back to smaller clusters when the preferred one would not give every CTA an SM of its own
    // (C3 with clusters of 8: 256 CTAs on 148 SMs 3.64 ms, clusters of 4: 128 CTAs 3.05 ms); the second pass takes
    // whatever exists.
    const int cs32 = pr.D <= 64 ? 1 : ((pr.D % 32 == 0 && pr.D / 32 <= 8) ? pr.D / 32 : 0);
    for (int pass = 0; pass < 2; ++pass)
      for (int ci = -1; ci < 8; ++ci) {
        // (large batches of the single-gate cell do best without any cluster: Elman B1024 D=128, one CTA per head 100 M
        // tokens/s, clusters of 2 x 64 units 70)
        if (ci < 0 && (want_cs || streamed(pr) || !cs32 || (fill && cd.Gr < 3))) continue;
        int cs = ci < 0 ? cs32 : (want_cs ? want_cs : (fill ? order_large[ci] : order_small[ci]));
        if (ci >= 0 && !fill && !want_cs && cs32 && cs > cs32) continue;  // fewer than 32 units per CTA
        if (streamed(pr) && !want_cs) cs = pr.D / kStreamU;  // the streamed kernels have one geometry
        const bool crowded = !fill && !want_cs && !streamed(pr) && pairs * cs > sms;
        if (!(pass == 0 && crowded) && tile_ok(pr, cd, cs, bt)) { *cs_out = cs; *bt_out = bt; return true; }
        if (want_cs || streamed(pr)) break;
      }
    if (want_bt) break;
  }
  return false;
}

static int validate_problem(const frnn_problem* pr, CellDims* cd) {
  if (!pr) return FRNN_ERR_NULL;
  if (!cell_dims(pr->cell, cd)) return FRNN_ERR_CELL;
  constexpr int io = kF16 ? FRNN_DTYPE_F16 : FRNN_DTYPE_BF16;  // the element type this build of the kernels computes in
  if (pr->dtype_io != io) return FRNN_ERR_DTYPE;
  if (pr->dtype_state != io && pr->dtype_state != FRNN_DTYPE_F32) return FRNN_ERR_DTYPE;
  if (pr->B < 1 || pr->T < 1 || pr->N < 1 || pr->D < 1) return FRNN_ERR_SHAPE;
  if (pr->N > 65535) return FRNN_ERR_SHAPE;
  if (pr->D % 16) return FRNN_ERR_SHAPE;
  bool kt_ok = pr->D > 256 && pr->D <= kStreamMaxD && pr->D % kStreamU == 0;  // streamed kernels
  for (int i = 0; i < kNumKT; ++i) kt_ok = kt_ok || (kKTs[i] * 16 == pr->D);
  if (!kt_ok) return FRNN_ERR_SHAPE;
  return FRNN_OK;
}

static int fill_plan(const frnn_problem* pr, int cs, int bt, int stages, frnn_plan* out) {
  CellDims cd;
  const int rc = validate_problem(pr, &cd);
  if (rc) return rc;
  if (!out) return FRNN_ERR_NULL;
  if (stages != 0 && stages != kStages) return FRNN_ERR_PLAN;
  int ccs = 0, cbt = 0;
  if (!choose_tile(*pr, cd, cs, bt, &ccs, &cbt)) return (cs || bt) ? FRNN_ERR_PLAN : FRNN_ERR_SHAPE;
  if ((long long)((pr->B + cbt - 1) / cbt) > 65535) return FRNN_ERR_SHAPE;
  frnn_plan pl = {};
  pl.abi_version = FRNN_ABI_VERSION;
  pl.prob = *pr;
  pl.cluster_size = ccs;
  pl.units_per_cta = pr->D / ccs;
  pl.batch_tile = cbt;
  pl.threads = plan_threads(cd, pl.units_per_cta, cbt);
  pl.wx_stages = kStages;
  // measured on B200: LSTM B1024 T512 N16 D64 (128 CTAs of 128 rows) forward loop 2.07 ms against 3.40 ms on the 16-row
  // tiles; B512 T128 N16 (64 CTAs) 0.49 against 0.51 ms -- a step of the 128-row loop takes ~3.8 us however few CTAs run,
  // so it pays once its CTAs occupy most of the SMs.  GRU B1024 T512 N16 D64: 1.74 against 3.25 ms.
  pl.wide_forward = wide_gates_problem(*pr) && ccs == 1 && cbt == 16 &&
                    (bt == kWideBatchTile || (!cs && !bt && (long long)(pr->B / kWideBatchTile) * pr->N >= 96));
  pl.cache_slots = cache_slots_of(*pr, cd);
  // one bf16 pair per (item, slot, step) in the time loops' own order; batch rows padded to whole tiles
  const uint64_t rows = (uint64_t)((pr->B + cbt - 1) / cbt) * cbt;
  pl.cache_bytes = rows * pr->T * pl.cache_slots * pr->N * pr->D * 2;
  const WsLayout w = workspace_layout(*pr, cd);
  pl.workspace_bytes = w.total;
  pl.grads_offset = w.grads;
  pl.grads_count = (uint64_t)cd.Gr * pr->N * pr->D * pr->D + (uint64_t)cd.Gt * pr->N * pr->D;
  *out = pl;
  return FRNN_OK;
}

static int check_plan(const frnn_plan* pl, CellDims* cd) {
  if (!pl) return FRNN_ERR_NULL;
  if (pl->abi_version != FRNN_ABI_VERSION) return FRNN_ERR_PLAN;
  const int rc = validate_problem(&pl->prob, cd);
  if (rc) return rc;
  if (!tile_ok(pl->prob, *cd, pl->cluster_size, pl->batch_tile)) return FRNN_ERR_PLAN;
  if (pl->units_per_cta * pl->cluster_size != pl->prob.D) return FRNN_ERR_PLAN;
  if (pl->threads != plan_threads(*cd, pl->units_per_cta, pl->batch_tile)) return FRNN_ERR_PLAN;
  if (pl->workspace_bytes != workspace_layout(pl->prob, *cd).total) return FRNN_ERR_PLAN;
  if (pl->wide_forward && !(pl->wide_forward == 1 && wide_gates_problem(pl->prob) && pl->cluster_size == 1 && pl->batch_tile == 16))
    return FRNN_ERR_PLAN;
  return FRNN_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Strides of a caller-produced tensor: all zero = dense (the defaults are filled in), else each a non-negative
// multiple of 8 elements (16 bytes: what the 4/8-byte cp.async reads and the tensor maps need).
static bool resolve_strides(const int64_t (&in)[4], const long long (&dense)[4], long long (&out)[4]) {
  if (!in[0] && !in[1] && !in[2] && !in[3]) {
    for (int i = 0; i < 4; ++i) out[i] = dense[i];
    return true;
  }
  for (int i = 0; i < 4; ++i) {
    if (in[i] < 0 || in[i] % 8) return false;
    out[i] = in[i];
  }
  return true;
}

static cudaError_t launch_loop(const LoopKernel& k, const frnn_plan& pl, const LoopParams& lp, cudaStream_t stream) {
  const size_t smem = k.smem_bytes(pl.prob.D, pl.units_per_cta, pl.threads);
  // always the fixed maximum, never this plan's own size: the attribute belongs to the kernel, not to the launch, and a
  // second host thread launching the same instantiation with a larger tile must not find it lowered in between
  cudaError_t e = cudaFuncSetAttribute(k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem);
  if (e != cudaSuccess) return e;
  if (pl.cluster_size > 8) {  // clusters of more than 8 CTAs are a non-portable size: opt in
    e = cudaFuncSetAttribute(k.fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)pl.cluster_size, (unsigned)((pl.prob.B + pl.batch_tile - 1) / pl.batch_tile), (unsigned)pl.prob.N);
  cfg.blockDim = dim3((unsigned)pl.threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)pl.cluster_size;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pl.cluster_size > 1 ? 1 : 0;
  void* args[1] = {const_cast<LoopParams*>(&lp)};
  return cudaLaunchKernelExC(&cfg, k.fn, args);
}

static int sm_count_cached() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev] = v;
  }
  return cached[dev];
}

}  // namespace FRNN_NS

using namespace FRNN_NS;

// This file is compiled twice (see frnn_elem.cuh).  The bfloat16 build owns the public names and forwards float16
// problems to the float16 build, whose entry points carry the suffix _f16 and stay private to the library.
#ifdef FRNN_F16
#define FRNN_ENTRY(name) __attribute__((visibility("hidden"))) name##_f16
#define FRNN_FORWARD_F16(is_f16, call)
#else
#define FRNN_ENTRY(name) name
#define FRNN_FORWARD_F16(is_f16, call) \
  if (is_f16) return call
extern "C" {
int frnn_query_f16(const frnn_problem*, frnn_plan*);
int frnn_query_tile_f16(const frnn_problem*, int, int, int, frnn_plan*);
int frnn_forward_f16(const frnn_plan*, const frnn_fwd_args*, void*);
int frnn_backward_parts_f16(const frnn_plan*, const frnn_bwd_args*, void*, int);
int frnn_finalize_grads_f16(const frnn_plan*, const void*, void*, void*, void*);
}
#endif
// float32 problems (Wx, R, b, states and gradients all fp32) go to the float32 loops of frnn_f32.cu
#ifdef FRNN_F16
#define FRNN_FORWARD_F32(is_f32, call)
#else
#define FRNN_FORWARD_F32(is_f32, call) \
  if (is_f32) return call
extern "C" {
int frnn_query_f32(const frnn_problem*, int, int, int, frnn_plan*);
int frnn_forward_f32(const frnn_plan*, const frnn_fwd_args*, void*);
int frnn_backward_parts_f32(const frnn_plan*, const frnn_bwd_args*, void*, int);
int frnn_finalize_grads_f32(const frnn_plan*, const void*, void*, void*, void*);
}
#endif
static inline bool wants_f32(const frnn_problem* pr) { return pr && pr->dtype_io == FRNN_DTYPE_F32; }
static inline bool wants_f32(const frnn_plan* pl) { return pl && pl->prob.dtype_io == FRNN_DTYPE_F32; }
static inline bool wants_f16(const frnn_problem* pr) { return pr && pr->dtype_io == FRNN_DTYPE_F16; }
static inline bool wants_f16(const frnn_plan* pl) { return pl && pl->prob.dtype_io == FRNN_DTYPE_F16; }

extern "C" {

#ifndef FRNN_F16
int frnn_abi_version(void) { return FRNN_ABI_VERSION; }
#endif

int FRNN_ENTRY(frnn_query)(const frnn_problem* problem, frnn_plan* out) {
  FRNN_FORWARD_F32(wants_f32(problem), frnn_query_f32(problem, 0, 0, 0, out));
  FRNN_FORWARD_F16(wants_f16(problem), frnn_query_f16(problem, out));
  return fill_plan(problem, 0, 0, 0, out);
}

int FRNN_ENTRY(frnn_query_tile)(const frnn_problem* problem, int cluster_size, int batch_tile, int wx_stages, frnn_plan* out) {
  FRNN_FORWARD_F32(wants_f32(problem), frnn_query_f32(problem, cluster_size, batch_tile, wx_stages, out));
  FRNN_FORWARD_F16(wants_f16(problem), frnn_query_tile_f16(problem, cluster_size, batch_tile, wx_stages, out));
  return fill_plan(problem, cluster_size, batch_tile, wx_stages, out);
}

int FRNN_ENTRY(frnn_forward)(const frnn_plan* plan, const frnn_fwd_args* a, void* stream_) {
  FRNN_FORWARD_F32(wants_f32(plan), frnn_forward_f32(plan, a, stream_));
  FRNN_FORWARD_F16(wants_f16(plan), frnn_forward_f16(plan, a, stream_));
  CellDims cd;
  int rc = check_plan(plan, &cd);
  if (rc) return rc;
  if (!a || !a->Wx || !a->R || !a->b || !a->s0 || !a->states || !a->workspace) return FRNN_ERR_NULL;
  const frnn_problem& pr = plan->prob;
  if (pr.training && cache_slots_of(pr, cd) > 0 && !a->cache) return FRNN_ERR_NULL;
  if (!aligned16(a->Wx) || !aligned16(a->R) || !aligned16(a->b) || !aligned16(a->s0) || !aligned16(a->states) ||
      !aligned16(a->workspace) || (a->cache && !aligned16(a->cache)))
    return FRNN_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const WsLayout w = workspace_layout(pr, cd);
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  const long long nd = (long long)pr.N * pr.D;
  const long long wx_dense[4] = {(long long)pr.T * cd.Gw * nd, cd.Gw * nd, nd, pr.D};
  long long wxs[4];
  if (!resolve_strides(a->wx_stride, wx_dense, wxs)) return FRNN_ERR_ALIGN;

  // keep_packed_r: the workspace is left as the previous call left it (R fragments kept, status block not cleared, so
  // an expired wait of an earlier step stays on record until the caller reads it)
  cudaError_t e = plan->keep_packed_r ? cudaSuccess : cudaMemsetAsync(ws, 0, kStatusBytes, stream);
  if (e != cudaSuccess) return (int)e;
  if (a->last && !aligned16(a->last)) return FRNN_ERR_ALIGN;
  // `last`: one strided device copy of states[:, :, T-1] behind the time loop.  (Storing it from inside the forward
  // kernel, after the loop, cost the C2 forward loop 6 %: the longer live ranges changed its register allocation.)
  auto copy_last = [&]() -> cudaError_t {
    if (!a->last) return cudaSuccess;
    const size_t row = (size_t)pr.N * pr.D * (pr.dtype_state == FRNN_DTYPE_F32 ? 4 : 2);
    return cudaMemcpy2DAsync(a->last, row, static_cast<const unsigned char*>(a->states) + (size_t)(pr.T - 1) * row,
                             (size_t)pr.T * row, row, (size_t)cd.S * pr.B, cudaMemcpyDeviceToDevice, stream);
  };
  if (is_wide(*plan)) {
    if (plan->probe_noop_cell) return FRNN_ERR_PLAN;
    e = launch_wide_forward(a->Wx, wxs[0], wxs[1], wxs[3], a->R, a->b, a->s0, a->states, reinterpret_cast<unsigned*>(ws), pr.B,
                            pr.T, pr.N, plan->test_drop_exchange, stream);
    return (int)(e == cudaSuccess ? copy_last() : e);
  }
  if (plan->wide_forward) {  // LSTM / GRU, head dim 64: 128-row forward loop; cache in the layout of the reverse loop's tile
    if (plan->probe_noop_cell) return FRNN_ERR_PLAN;
    e = launch_wide_gates_forward(pr.cell, a->Wx, wxs[0], wxs[1], wxs[2], wxs[3], a->R, a->b, a->s0, a->states, pr.training ? a->cache : nullptr,
                                 reinterpret_cast<unsigned*>(ws), pr.B, pr.T, pr.N, pr.forward_clip, plan->test_drop_exchange, stream);
    return (int)(e == cudaSuccess ? copy_last() : e);
  }
  if (!plan->keep_packed_r) e = launch_pack_recurrent(a->R, ws + w.rpack_fwd, cd.Gr, pr.N, pr.D, 0, stream);
  if (e != cudaSuccess) return (int)e;

  LoopParams lp = {};
  lp.Wx = static_cast<const elem_t*>(a->Wx);
  lp.Rpack = reinterpret_cast<const uint4*>(ws + w.rpack_fwd);
  lp.bias = static_cast<const elem_t*>(a->b);
  lp.s0 = a->s0;
  lp.states = a->states;
  lp.cache = pr.training ? static_cast<elem_t*>(a->cache) : nullptr;
  lp.status = reinterpret_cast<unsigned*>(ws);
  lp.B = pr.B; lp.T = pr.T; lp.N = pr.N; lp.D = pr.D;
  lp.U = plan->units_per_cta; lp.CS = plan->cluster_size;
  lp.state_f32 = pr.dtype_state == FRNN_DTYPE_F32;
  lp.fclip = pr.forward_clip; lp.gclip = pr.grad_clip; lp.grad_cut = pr.grad_cut;
  lp.test_drop = plan->test_drop_exchange;
  lp.wx_sb = wxs[0]; lp.wx_st = wxs[1]; lp.wx_sg = wxs[2]; lp.wx_sn = wxs[3];
  const LoopKernel k = plan->probe_noop_cell ? get_fwd_kernel_floor(kernel_cell(pr), kernel_kt(pr), plan->batch_tile / 8)
                                             : get_fwd_kernel(kernel_cell(pr), kernel_kt(pr), plan->batch_tile / 8);
  if (!k.fn) return FRNN_ERR_PLAN;
  e = launch_loop(k, *plan, lp, stream);
  return (int)(e == cudaSuccess ? copy_last() : e);
}

#ifndef FRNN_F16
int frnn_backward(const frnn_plan* plan, const frnn_bwd_args* a, void* stream_) {
  return frnn_backward_parts(plan, a, stream_, FRNN_PART_LOOP | FRNN_PART_DR);
}
#endif

int FRNN_ENTRY(frnn_backward_parts)(const frnn_plan* plan, const frnn_bwd_args* a, void* stream_, int parts) {
  FRNN_FORWARD_F32(wants_f32(plan), frnn_backward_parts_f32(plan, a, stream_, parts));
  FRNN_FORWARD_F16(wants_f16(plan), frnn_backward_parts_f16(plan, a, stream_, parts));
  CellDims cd;
  int rc = check_plan(plan, &cd);
  if (rc) return rc;
  const frnn_problem& pr = plan->prob;
  if (!pr.training) return FRNN_ERR_TRAINING;
  if (!a || !a->R || !a->s0 || !a->states || !a->dstates || !a->dWx || !a->ds0 || !a->workspace) return FRNN_ERR_NULL;
  if (cache_slots_of(pr, cd) > 0 && !a->cache) return FRNN_ERR_NULL;
  if (!aligned16(a->R) || !aligned16(a->s0) || !aligned16(a->states) || !aligned16(a->dstates) || !aligned16(a->dWx) ||
      !aligned16(a->ds0) || !aligned16(a->workspace) || (a->cache && !aligned16(a->cache)))
    return FRNN_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const WsLayout w = workspace_layout(pr, cd);
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  float* grads = reinterpret_cast<float*>(ws + w.grads);
  const size_t nR = (size_t)cd.Gr * pr.N * pr.D * pr.D, nb = (size_t)cd.Gt * pr.N * pr.D;
  const long long nd = (long long)pr.N * pr.D;
  const long long ds_dense[4] = {(long long)pr.B * pr.T * nd, (long long)pr.T * nd, nd, pr.D};
  long long dss[4];
  if (!resolve_strides(a->dstates_stride, ds_dense, dss)) return FRNN_ERR_ALIGN;

  cudaError_t e = cudaSuccess;
  if (parts & FRNN_PART_LOOP) {
    e = cudaMemsetAsync(ws, 0, kStatusBytes, stream);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemsetAsync(grads, 0, (nR + nb) * sizeof(float), stream);
    if (e != cudaSuccess) return (int)e;
    if (!is_wide(*plan)) e = launch_pack_recurrent(a->R, ws + w.rpack_bwd, cd.Gr, pr.N, pr.D, 1, stream);
    if (e != cudaSuccess) return (int)e;
  }
  if (is_wide(*plan)) {  // one kernel: reverse loop with dR and db accumulated inside; the dR part has nothing left to do
    if (plan->probe_noop_cell) return FRNN_ERR_PLAN;
    if (parts & FRNN_PART_LOOP)
      e = launch_wide_backward(a->R, a->s0, a->states, a->dstates, dss[1], dss[2], dss[3], a->dWx, a->ds0, grads, grads + nR,
                               reinterpret_cast<unsigned*>(ws), pr.B, pr.T, pr.N, plan->test_drop_exchange, stream);
    return (int)e;
  }

  LoopParams lp = {};
  lp.Rpack = reinterpret_cast<const uint4*>(ws + w.rpack_bwd);
  lp.s0 = a->s0;
  lp.states = const_cast<void*>(a->states);
  lp.cache = static_cast<elem_t*>(const_cast<void*>(a->cache));
  lp.dstates = a->dstates;
  lp.dWx = static_cast<elem_t*>(a->dWx);
  lp.dg0 = reinterpret_cast<elem_t*>(ws + w.dg0);
  lp.ds0 = a->ds0;
  lp.dbias = grads + nR;
  lp.status = reinterpret_cast<unsigned*>(ws);
  lp.B = pr.B; lp.T = pr.T; lp.N = pr.N; lp.D = pr.D;
  lp.U = plan->units_per_cta; lp.CS = plan->cluster_size;
  lp.state_f32 = pr.dtype_state == FRNN_DTYPE_F32;
  lp.fclip = pr.forward_clip; lp.gclip = pr.grad_clip; lp.grad_cut = pr.grad_cut;
  lp.test_drop = plan->test_drop_exchange;
  lp.ds_ss = dss[0]; lp.ds_sb = dss[1]; lp.ds_st = dss[2]; lp.ds_sn = dss[3];
  if (parts & FRNN_PART_LOOP) {
    const int mpw = bwd_mpw(pr, cd, plan->cluster_size, plan->batch_tile);
    const LoopKernel k = plan->probe_noop_cell ? get_bwd_kernel_floor(kernel_cell(pr), kernel_kt(pr), plan->batch_tile / 8, mpw)
                                               : get_bwd_kernel(kernel_cell(pr), kernel_kt(pr), plan->batch_tile / 8, mpw);
    if (!k.fn) return FRNN_ERR_PLAN;
    e = launch_loop(k, *plan, lp, stream);
    if (e != cudaSuccess) return (int)e;
  }
  // measured on B200: the tcgen05 kernel wins from head_dim 128 up (C2 0.167 vs 0.212 ms, C3 0.263 vs 0.304 ms) and at
  // head_dim 64 when the gates fill two 128-row tiles (LSTM B1024 T512 N16 D64: 1.43 vs 1.60 ms; the GRU's 192 rows, one
  // and a half tiles, lose: 1.43 vs 1.25 ms); for the one-gate Elman
  // cell at head_dim 64 (half a tile) the warp-MMA kernel with its many small CTAs streams faster (C5 1.55 vs 3.1 ms)
  // (the tcgen05 kernel keeps a whole row tile of dR, N = D <= 256 columns, in one TMEM allocation)
  if ((parts & FRNN_PART_DR) && (pr.D >= 128 || cd.Gr * pr.D >= 256) && recurrent_grad_tma_supported(pr.D, lp.state_f32))
    // bf16 states: both operands are [64 steps][64] tiles a tensor-map copy delivers ready for the MMA (C2: 0.087 ms
    // against 0.167 ms for the cp.async-fed kernel below)
    e = launch_recurrent_grad_tma(pr.cell, pr.B, pr.T, pr.N, pr.D, cd.Gr, cd.Gw, a->dWx, ws + w.dg0, a->states, a->s0, grads,
                                  reinterpret_cast<unsigned*>(ws), sm_count_cached(), stream);
  else if ((parts & FRNN_PART_DR) && pr.D >= 128 && pr.D <= 256)
    e = launch_recurrent_grad_tc(pr.cell, pr.B, pr.T, pr.N, pr.D, cd.Gr, cd.Gw, lp.state_f32, a->dWx, ws + w.dg0, a->states,
                                 a->s0, grads, reinterpret_cast<unsigned*>(ws), sm_count_cached(), stream);
  else if (parts & FRNN_PART_DR)
    e = launch_recurrent_grad(pr.cell, pr.B, pr.T, pr.N, pr.D, cd.Gr, cd.Gw, lp.state_f32, a->dWx, ws + w.dg0, a->states,
                            a->s0, grads, sm_count_cached(), stream);
  return (int)e;
}

int FRNN_ENTRY(frnn_finalize_grads)(const frnn_plan* plan, const void* grads_f32, void* dR, void* db, void* stream_) {
  FRNN_FORWARD_F32(wants_f32(plan), frnn_finalize_grads_f32(plan, grads_f32, dR, db, stream_));
  FRNN_FORWARD_F16(wants_f16(plan), frnn_finalize_grads_f16(plan, grads_f32, dR, db, stream_));
  CellDims cd;
  int rc = check_plan(plan, &cd);
  if (rc) return rc;
  if (!grads_f32 || !dR || !db) return FRNN_ERR_NULL;
  const frnn_problem& pr = plan->prob;
  const size_t nR = (size_t)cd.Gr * pr.N * pr.D * pr.D, nb = (size_t)cd.Gt * pr.N * pr.D;
  return (int)launch_cast_grads(static_cast<const float*>(grads_f32), dR, db, nR, nb, static_cast<cudaStream_t>(stream_));
}

#ifndef FRNN_F16
int frnn_read_device_status(const void* workspace, void* stream_, frnn_dev_status* out) {
  if (!workspace || !out) return FRNN_ERR_NULL;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemcpyAsync(out, workspace, sizeof(frnn_dev_status), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);
}

const char* frnn_status_string(int code) {
  switch (code) {
    case FRNN_OK: return "ok";
    case FRNN_ERR_NULL: return "frnn: a required pointer is NULL";
    case FRNN_ERR_CELL: return "frnn: unknown cell (expected lstm, gru, elman or slstm)";
    case FRNN_ERR_SHAPE: return "frnn: unsupported shape (B,T,N >= 1; head_dim in {16,32,64,96,128,192,256} or a multiple of 64 up to 1024; float32: a multiple of 4 up to 1024)";
    case FRNN_ERR_DTYPE: return "frnn: unsupported dtype (Wx/R/b bfloat16 or float16 with states of the same type or float32; or everything float32)";
    case FRNN_ERR_ALIGN: return "frnn: tensor pointers must be 16-byte aligned";
    case FRNN_ERR_PLAN: return "frnn: invalid plan or tile for this problem";
    case FRNN_ERR_TRAINING: return "frnn: backward needs a plan made with training = 1";
    case FRNN_ERR_DEVICE: return "frnn: no sm_100 device / kernel image";
    case FRNN_ERR_TOO_LARGE: return "frnn: size beyond the fixed limit of this entry point";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "frnn: unknown status";
}
#endif

}  // extern "C"
