// Host-side launchers shared by the translation units of libfrnn_b200.so.
#pragma once
#include "frnn_common.cuh"

namespace FRNN_NS {

// head dims (D = 16*KT) and batch tiles (BT = 8*NT) the time-loop kernels are instantiated for
#define FRNN_FOREACH_KT(X, ...) X(1, __VA_ARGS__) X(2, __VA_ARGS__) X(4, __VA_ARGS__) X(6, __VA_ARGS__) X(8, __VA_ARGS__) X(12, __VA_ARGS__) X(16, __VA_ARGS__)
constexpr int kNumKT = 7;
constexpr int kKTs[kNumKT] = {1, 2, 4, 6, 8, 12, 16};
constexpr int kNumNT = 3;
constexpr int kNTs[kNumNT] = {1, 2, 4};

// head dims above 256 (multiples of 64 up to kStreamMaxD) run the streamed kernels: kStreamKT k-steps of R per warp
// in registers, U = kStreamU units per CTA, cluster size D / kStreamU (up to 16, non-portable above 8)
// (kStreamKT, kStreamU, kStreamMaxD: frnn_common.cuh)

struct LoopKernel {
  const void* fn;      // kernel entry
  int max_threads;     // __launch_bounds__ of the instantiation
  size_t (*smem_bytes)(int D, int U, int threads);
};

// defined once per (cell, direction) in frnn_inst_*.cu; returns fn == nullptr when not instantiated
LoopKernel get_fwd_kernel(int cell, int kt, int nt);
LoopKernel get_bwd_kernel(int cell, int kt, int nt, int mpw);  // mpw = 0: all-gather exchange, > 0: reduce-scatter
LoopKernel get_fwd_kernel_lstm(int kt, int nt);
LoopKernel get_fwd_kernel_gru(int kt, int nt);
LoopKernel get_fwd_kernel_elman(int kt, int nt);
LoopKernel get_fwd_kernel_slstm(int kt, int nt);
LoopKernel get_fwd_kernel_elmanc(int kt, int nt);
LoopKernel get_bwd_kernel_elmanc(int kt, int nt, int mpw);
LoopKernel get_bwd_kernel_lstm(int kt, int nt, int mpw);
LoopKernel get_bwd_kernel_gru(int kt, int nt, int mpw);
LoopKernel get_bwd_kernel_elman(int kt, int nt, int mpw);
LoopKernel get_bwd_kernel_slstm(int kt, int nt, int mpw);

// chain-floor variants (frnn_inst_floor.cu); fn == nullptr for any tile but the benchmark configurations
LoopKernel get_fwd_kernel_floor(int cell, int kt, int nt);
LoopKernel get_bwd_kernel_floor(int cell, int kt, int nt, int mpw);

cudaError_t launch_pack_recurrent(const void* R, void* out, int Gr, int N, int D, int transpose, cudaStream_t stream);
cudaError_t launch_recurrent_grad(int cell, int B, int T, int N, int D, int Gr, int Gw, int state_f32, const void* dWx,
                                  const void* dg0, const void* states, const void* s0, float* dR, int sm_count,
                                  cudaStream_t stream);
cudaError_t launch_recurrent_grad_tc(int cell, int B, int T, int N, int D, int Gr, int Gw, int state_f32, const void* dWx,
                                     const void* dg0, const void* states, const void* s0, float* dR, unsigned* status,
                                     int sm_count, cudaStream_t stream);
// 128-row tensor-core time loops (frnn_wide.cu): one CTA per (head, 128 batch rows); the backward also produces dR and db
constexpr int kWideBatchTile = 128;
constexpr int kWideThreads = 160;
bool wide_supported(int cell, int D, int state_f32, float fclip, float gclip, int grad_cut);
// wx_s* / ds_s*: element strides of the batch, time and head dimensions of Wx / dstates (their head dim is contiguous)
cudaError_t launch_wide_forward(const void* Wx, long long wx_sb, long long wx_st, long long wx_sn, const void* R,
                                const void* bias, const void* s0, void* states, unsigned* status, int B, int T, int N,
                                int test_drop, cudaStream_t stream);
cudaError_t launch_wide_backward(const void* R, const void* s0, const void* states, const void* dstates, long long ds_sb,
                                 long long ds_st, long long ds_sn, void* dWx, void* ds0, float* dR, float* dbias,
                                 unsigned* status, int B, int T, int N, int test_drop, cudaStream_t stream);
// 128-row forward loop of the LSTM and GRU cells at head dim 64 (frnn_wide.cu); writes the activation cache in the layout of the
// cluster kernels' tile (1 CTA per head, 16 batch rows), which runs the reverse loop
bool wide_gates_forward_supported(int cell, int D, int state_f32);
cudaError_t launch_wide_gates_forward(int cell, const void* Wx, long long wx_sb, long long wx_st, long long wx_sg, long long wx_sn, const void* R,
                                     const void* bias, const void* s0, void* states, void* cache, unsigned* status, int B, int T,
                                     int N, float fclip, int test_drop, cudaStream_t stream);
// dR fed by tensor-map bulk copies (frnn_dr_tma.cu): bf16 states, head dims 64 .. 256 in steps of 64
bool recurrent_grad_tma_supported(int D, int state_f32);
cudaError_t launch_recurrent_grad_tma(int cell, int B, int T, int N, int D, int Gr, int Gw, const void* dWx, const void* dg0,
                                      const void* states, const void* s0, float* dR, unsigned* status, int sm_count,
                                      cudaStream_t stream);
cudaError_t launch_cast_grads(const float* src, void* dR, void* db, size_t nR, size_t nb, cudaStream_t stream);

}  // namespace FRNN_NS
