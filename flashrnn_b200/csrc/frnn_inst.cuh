// Instantiation helper: each frnn_inst_<dir>_<cell>.cu defines FRNN_INST_CELL / FRNN_INST_BWD / FRNN_INST_NAME
// and includes this file, which emits the kernels for every (KT, NT) and the lookup function.
//
// Lookup key: kt = head_dim / 16 for the register-resident kernels (head_dim <= 256); kt = 0 selects the streamed
// kernel for larger head dims (kStreamKT k-steps in registers, the rest re-read from L2 every step).
#include "frnn_aux.cuh"
#include "frnn_bwd.cuh"
#include "frnn_fwd.cuh"

namespace FRNN_NS {

#if FRNN_INST_BWD

template <int KT, int NT, int MPW, bool DYN>
static LoopKernel make_entry() {
  LoopKernel k;
  k.fn = reinterpret_cast<const void*>(&frnn_bwd_kernel<FRNN_INST_CELL, KT, NT, MPW, DYN>);
  k.smem_bytes = [](int D, int U, int threads) -> size_t { return bwd_smem_bytes<FRNN_INST_CELL, NT, MPW>(D, U, threads); };
  k.max_threads = LaunchBounds<FRNN_INST_CELL, KT>::threads;
  return k;
}
// reduce-scatter variants exist only where the geometry works out (CS = MPW * Gr <= 8, U a power of two times 16)
template <int KT, int NT, int MPW, bool V = RsGeom<FRNN_INST_CELL, KT, MPW>::valid>
struct RsEntry { static LoopKernel get() { return LoopKernel{nullptr, 0, nullptr}; } };
template <int KT, int NT, int MPW>
struct RsEntry<KT, NT, MPW, true> { static LoopKernel get() { return make_entry<KT, NT, MPW, false>(); } };

LoopKernel FRNN_INST_NAME(int kt, int nt, int mpw) {
  if (kt == 0 && mpw == 0) {
    if (nt == 1) return make_entry<kStreamKT, 1, 0, true>();
    if (nt == 2) return make_entry<kStreamKT, 2, 0, true>();
    return LoopKernel{nullptr, 0, nullptr};
  }
#define FRNN_CASE(KT, NT) if (kt == KT && nt == NT && mpw == 0) return make_entry<KT, NT, 0, false>();
#define FRNN_RS(KT, NT, MPW) if (kt == KT && nt == NT && mpw == MPW) return RsEntry<KT, NT, MPW>::get();
#define FRNN_ROW(KT, unused)                                                                     \
  FRNN_CASE(KT, 1) FRNN_CASE(KT, 2) FRNN_CASE(KT, 4)                                             \
  FRNN_RS(KT, 1, 1) FRNN_RS(KT, 1, 2) FRNN_RS(KT, 1, 4) FRNN_RS(KT, 1, 8)                        \
  FRNN_RS(KT, 2, 1) FRNN_RS(KT, 2, 2) FRNN_RS(KT, 2, 4) FRNN_RS(KT, 2, 8)
  FRNN_FOREACH_KT(FRNN_ROW, 0)
#undef FRNN_ROW
#undef FRNN_RS
#undef FRNN_CASE
  return LoopKernel{nullptr, 0, nullptr};
}

#else

template <int KT, int NT, bool DYN>
static LoopKernel make_entry() {
  LoopKernel k;
  k.fn = reinterpret_cast<const void*>(&frnn_fwd_kernel<FRNN_INST_CELL, KT, NT, DYN>);
  k.smem_bytes = [](int D, int U, int threads) -> size_t { return fwd_smem_bytes<FRNN_INST_CELL, NT>(D, U, threads); };
  k.max_threads = LaunchBounds<FRNN_INST_CELL, KT>::threads;
  return k;
}

LoopKernel FRNN_INST_NAME(int kt, int nt) {
  if (kt == 0) {
    if (nt == 1) return make_entry<kStreamKT, 1, true>();
    if (nt == 2) return make_entry<kStreamKT, 2, true>();
    return LoopKernel{nullptr, 0, nullptr};
  }
#define FRNN_CASE(KT, NT) if (kt == KT && nt == NT) return make_entry<KT, NT, false>();
#define FRNN_ROW(KT, unused) FRNN_CASE(KT, 1) FRNN_CASE(KT, 2) FRNN_CASE(KT, 4)
  FRNN_FOREACH_KT(FRNN_ROW, 0)
#undef FRNN_ROW
#undef FRNN_CASE
  return LoopKernel{nullptr, 0, nullptr};
}

#endif

}  // namespace FRNN_NS
