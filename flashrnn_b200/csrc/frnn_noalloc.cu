// frnn_forward_noalloc: the forward pass for callers that cannot provide a workspace.
//
// Some hosts of this library may not allocate device memory at the point where they call it: a serving loop
// whose memory pool was sized and handed out at start-up, code that runs while a CUDA graph is being captured,
// or an embedding runtime that forbids cudaMalloc on its hot path because the call synchronises the device.
// For them the forward's scratch (status block + the recurrent matrix repacked into tensor-core fragments)
// lives in a fixed array inside the library image instead of a caller-provided workspace.
#ifndef FRNN_F16  // compiled once: frnn_query / frnn_forward below pick the kernels by frnn_problem.dtype_io
#include "../../include/frnn.h"

#include <cuda_runtime.h>

#include <mutex>

// The scratch itself.  Every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FRNN_NOALLOC_MAX_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

// In host code `g_noalloc_scratch` is only a handle of the device array, not an address a kernel could use:
// the device address is looked up once per device, with that device current.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return FRNN_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return FRNN_ERR_DEVICE;
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return FRNN_OK;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

extern "C" int frnn_forward_noalloc(const frnn_problem* problem, const frnn_fwd_args* args, void* stream) {
  if (!problem || !args) return FRNN_ERR_NULL;
  frnn_plan plan;
  const int rc = frnn_query(problem, &plan);
  if (rc != FRNN_OK) return rc;
  // what the forward touches of a workspace: the 256-byte status block followed by R repacked (same size as R).  Gate count of R: 4 (lstm, slstm), 3 (gru), 1 (elman).
  const size_t gr = problem->cell == FRNN_CELL_GRU ? 3 : (problem->cell == FRNN_CELL_ELMAN ? 1 : 4);
  const size_t esz = problem->dtype_io == FRNN_DTYPE_F32 ? 4 : 2;  // float32 problems keep a transposed fp32 copy of R there
  const size_t need = 256 + align_up(gr * (size_t)problem->N * problem->D * problem->D * esz, 256);
  if (need > (size_t)FRNN_NOALLOC_MAX_SCRATCH_BYTES) return FRNN_ERR_TOO_LARGE;
  unsigned char* scratch = nullptr;
  const int sc = scratch_for_current_device(&scratch);
  if (sc != FRNN_OK) return sc;
  frnn_fwd_args a = *args;
  a.workspace = scratch;  // frnn_forward clears the status block and rewrites the fragments on every call
  return frnn_forward(&plan, &a, stream);
}

#endif  // FRNN_F16
