// Instantiation helper: each frnn_inst_<dir>_<cell>.cu defines FRNN_INST_CELL / FRNN_INST_BWD / FRNN_INST_NAME
// and includes this file, which emits the kernels for every (KT, NT) and the lookup function.
#include "frnn_aux.cuh"
#include "frnn_bwd.cuh"
#include "frnn_fwd.cuh"

namespace frnn {

template <int KT, int NT>
static LoopKernel make_entry() {
  LoopKernel k;
#if FRNN_INST_BWD
  k.fn = reinterpret_cast<const void*>(&frnn_bwd_kernel<FRNN_INST_CELL, KT, NT>);
  k.smem_bytes = [](int U, int threads) -> size_t { return bwd_smem_bytes<FRNN_INST_CELL, KT, NT>(U, threads); };
#else
  k.fn = reinterpret_cast<const void*>(&frnn_fwd_kernel<FRNN_INST_CELL, KT, NT>);
  k.smem_bytes = [](int U, int threads) -> size_t { return fwd_smem_bytes<FRNN_INST_CELL, KT, NT>(U, threads); };
#endif
  k.max_threads = MaxThreads<KT>::v;
  return k;
}

LoopKernel FRNN_INST_NAME(int kt, int nt) {
#define FRNN_CASE(KT, NT) if (kt == KT && nt == NT) return make_entry<KT, NT>();
#define FRNN_ROW(KT, unused) FRNN_CASE(KT, 1) FRNN_CASE(KT, 2) FRNN_CASE(KT, 4)
  FRNN_FOREACH_KT(FRNN_ROW, 0)
#undef FRNN_ROW
#undef FRNN_CASE
  return LoopKernel{nullptr, 0, nullptr};
}

}  // namespace frnn
