// Measurement variants of the time-loop kernels: the tiles of the benchmark configurations with a pass-through in
// place of the gate arithmetic (CELL | kNoopCell).  frnn_plan.probe_noop_cell selects them; their step time is the
// floor of the serial chain (exchange wait, matrix product, barriers, copies) that no cell math can undercut.
#include "frnn_aux.cuh"
#include "frnn_bwd.cuh"
#include "frnn_fwd.cuh"

namespace FRNN_NS {

template <int CELL, int KT, int NT>
static LoopKernel floor_fwd() {
  LoopKernel k;
  k.fn = reinterpret_cast<const void*>(&frnn_fwd_kernel<CELL | kNoopCell, KT, NT, false>);
  k.smem_bytes = [](int D, int U, int threads) -> size_t { return fwd_smem_bytes<CELL, NT>(D, U, threads); };
  k.max_threads = LaunchBounds<CELL, KT>::threads;
  return k;
}
template <int CELL, int KT, int NT, int MPW>
static LoopKernel floor_bwd() {
  LoopKernel k;
  k.fn = reinterpret_cast<const void*>(&frnn_bwd_kernel<CELL | kNoopCell, KT, NT, MPW, false>);
  k.smem_bytes = [](int D, int U, int threads) -> size_t { return bwd_smem_bytes<CELL, NT, MPW>(D, U, threads); };
  k.max_threads = LaunchBounds<CELL, KT>::threads;
  return k;
}

// lstm head dim 256 (reduce-scatter backward, cluster of 8), gru head dim 128, slstm head dim 192; 8-row batch tiles
LoopKernel get_fwd_kernel_floor(int cell, int kt, int nt) {
  if (cell == CELL_LSTM && kt == 16 && nt == 1) return floor_fwd<CELL_LSTM, 16, 1>();
  if (cell == CELL_GRU && kt == 8 && nt == 1) return floor_fwd<CELL_GRU, 8, 1>();
  if (cell == CELL_SLSTM && kt == 12 && nt == 1) return floor_fwd<CELL_SLSTM, 12, 1>();
  return LoopKernel{nullptr, 0, nullptr};
}
LoopKernel get_bwd_kernel_floor(int cell, int kt, int nt, int mpw) {
  if (cell == CELL_LSTM && kt == 16 && nt == 1 && mpw == 2) return floor_bwd<CELL_LSTM, 16, 1, 2>();
  if (cell == CELL_GRU && kt == 8 && nt == 1 && mpw == 0) return floor_bwd<CELL_GRU, 8, 1, 0>();
  if (cell == CELL_SLSTM && kt == 12 && nt == 1 && mpw == 0) return floor_bwd<CELL_SLSTM, 12, 1, 0>();
  return LoopKernel{nullptr, 0, nullptr};
}

}  // namespace FRNN_NS
