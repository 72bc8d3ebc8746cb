/*
 * frnn.h -- C ABI of the B200-native FlashRNN recurrent hot path (libfrnn_b200.so).
 *
 * Plain C: pointers, sizes and PODs only (no torch / C++ types).  Every entry point states which
 * interface of the reference it replaces (paths are inside the reference project).
 *
 * Conventions
 *   - All tensor pointers are DEVICE pointers to dense row-major tensors in the reference's
 *     user-facing layouts (reference flashrnn/flashrnn/flashrnn.py:165-173):
 *         Wx[B,T,Gw,N,D]  R[Gr,N,D,D] (R[g,n,d_out,d_in])  b[Gt,N,D]
 *         s0[S,B,1,N,D]   states[S,B,T,N,D]   dstates like states   dWx like Wx   ds0 like s0
 *     The two large tensors the CALLER produces, Wx and dstates, may instead be strided views (element strides in
 *     frnn_fwd_args.wx_stride / frnn_bwd_args.dstates_stride): that covers the reference's other layout strings
 *     (input_shape "TBGHD", output_shape "STBHD", flashrnn.py:165-173, 291-321) without a permute + copy.  The tensors the
 *     library produces (states, dWx, ds0) are always dense; a caller that wants another order returns a permuted view.
 *   - The library never allocates or frees device memory and never synchronises the host with the
 *     device (except frnn_read_device_status, which copies one small struct back).  The caller provides
 *     the activation cache and a workspace whose sizes frnn_query reports.
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, in order.
 *   - Return value: 0 = OK; negative = host-side validation error (nothing was launched);
 *     positive = a CUDA runtime error code (cudaError_t) raised by a launch.
 *   - Re-entrant and thread-safe for distinct workspaces.
 */
#ifndef FRNN_H_
#define FRNN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FRNN_ABI_VERSION 3

/* cells: gate/state counts follow the reference registry flashrnn/flashrnn/flashrnn.py:49-71 */
enum { FRNN_CELL_LSTM = 0, FRNN_CELL_GRU = 1, FRNN_CELL_ELMAN = 2, FRNN_CELL_SLSTM = 3 };
enum { FRNN_DTYPE_BF16 = 0, FRNN_DTYPE_F32 = 1, FRNN_DTYPE_F16 = 2 };

/* status codes (negative = validation) */
enum {
  FRNN_OK = 0,
  FRNN_ERR_NULL = -1,          /* a required pointer is NULL */
  FRNN_ERR_CELL = -2,          /* unknown cell id */
  FRNN_ERR_SHAPE = -3,         /* B,T,N,D out of range / head_dim not supported */
  FRNN_ERR_DTYPE = -4,         /* unsupported dtype combination */
  FRNN_ERR_ALIGN = -5,         /* a pointer is not 16-byte aligned */
  FRNN_ERR_PLAN = -6,          /* plan does not belong to this problem / ABI version mismatch */
  FRNN_ERR_TRAINING = -7,      /* backward requested but the forward ran without a cache */
  FRNN_ERR_DEVICE = -8,        /* device is not sm_100 / kernel image missing */
  FRNN_ERR_TOO_LARGE = -9      /* size beyond a fixed limit of the entry point */
};

/* What to compute.  Replaces the shape/dtype part of the reference's FlashRNNConfig
 * (flashrnn/flashrnn/flashrnn.py:124-207) and the constructor arguments of the pybind class
 * FlashRNNFuncFused(training, batch_size, hidden_size, num_heads) (flashrnn/flashrnn/fused/flashrnn.cc:55-66). */
typedef struct frnn_problem {
  int32_t cell;          /* FRNN_CELL_*                                             */
  int32_t B, T, N, D;    /* batch, time steps, heads, head dim                     */
  int32_t dtype_io;      /* dtype of Wx, R, b, dWx, dR, db : FRNN_DTYPE_BF16 or _F16 (MMA operand type; accumulation and
                            gate math are fp32 either way), or FRNN_DTYPE_F32: the float32 loops (fp32 products on the
                            CUDA cores, exp-based nonlinearities; accurate to ~1e-5 against an fp32 reference, 4-5 x
                            slower than the 16-bit tensor-core loops; any head_dim % 4 == 0 up to 1024)              */
  int32_t dtype_state;   /* dtype of s0, states, dstates, ds0 : same as dtype_io, or F32 (F32 io needs F32 states) */
  int32_t training;      /* 1: forward writes the activation cache for backward     */
  float forward_clip;    /* > 0: clamp the new h to [-v, v]   (forward_clipval)     */
  float grad_clip;       /* > 0: clamp the recurrent dh to [-v, v] (gradient_recurrent_clipval) */
  int32_t grad_cut;      /* 1: drop the R^T delta term of dh_{t-1} in backward (gradient_recurrent_cut) */
} frnn_problem;

/* Launch plan chosen by frnn_query from the measured sm_100a tile table.  Replaces the reference's
 * compile-time tiling macros solved by flashrnn/autotune/constrint.py and bisected in
 * flashrnn/flashrnn/cuda_init_parametric.py:92-358.  Treat as opaque; sizes are for the caller. */
typedef struct frnn_plan {
  int32_t abi_version;
  frnn_problem prob;
  int32_t cluster_size;    /* CTAs that share one (head, batch tile); exchange h through DSMEM */
  int32_t units_per_cta;   /* hidden units of the head owned by one CTA                      */
  int32_t batch_tile;      /* batch rows per CTA (8, 16, 32 or 128; float32 loops: 8, 4 or 2) */
  int32_t threads;         /* threads per CTA of the time-loop kernels                       */
  int32_t wx_stages;       /* time steps of Wx prefetched ahead into shared memory           */
  int32_t cache_slots;     /* activation values cached per (b,t,n,d) in training             */
  int32_t test_drop_exchange; /* TEST HOOK, leave 0.  1: CTA 0 of every cluster withholds one exchange message
                                 (forward: its h of step 1; backward: its first message) so that its peers' bounded
                                 waits expire; the kernels then finish with invalid results and report it in the
                                 status block (float32 cluster loops: the message of step 1 in both loops).  With the 128-row loops (batch_tile 128, or wide_forward): one tile copy (step
                                 index 2) is announced to its barrier and never issued.  Exercises the failure-detection path
                                 without faulting the GPU.                                                          */
  int32_t keep_packed_r;      /* 0: frnn_forward clears the status block and repacks R into the workspace (default).
                                 1: the workspace is as an earlier frnn_forward with this plan left it and R has not
                                 changed since: skip both launches (step-by-step decoding calls frnn_forward once per
                                 token); a device status recorded by an earlier step stays until the caller reads it */
  int32_t probe_noop_cell;    /* MEASUREMENT HOOK, leave 0.  1: the time loops run with the gate arithmetic replaced by a
                                 pass-through (same exchange, matrix products, barriers and copies): their duration is
                                 the floor the serial chain of T dependent steps sets, which no cell math can undercut.
                                 Results are meaningless.  Exists for the tiles of the benchmark configurations only
                                 (lstm D=256, gru D=128, slstm D=192, 8-row batch tiles); elsewhere FRNN_ERR_PLAN.   */
  int32_t wide_forward;       /* 1: the forward loop runs as the 128-row tensor-core loop (tcgen05, one CTA per head and
                                 128 batch rows) while the reverse loop keeps the tile above, whose cache layout the
                                 forward loop writes.  Set by frnn_query for large-batch LSTM and GRU problems at
                                 head_dim 64 (16-bit states) on 16-row tiles; frnn_query_tile(cluster_size 1,
                                 batch_tile 128) asks for it, any other forced tile leaves it 0.                       */
  int32_t reserved[2];
  uint64_t cache_bytes;     /* size of the activation cache (opaque layout, tied to this plan) */
  uint64_t workspace_bytes; /* size of the scratch workspace                                  */
  uint64_t grads_offset;    /* byte offset, inside the workspace, of the fp32 gradients dR || db */
  uint64_t grads_count;     /* number of fp32 values there: Gr*N*D*D + Gt*N*D                 */
} frnn_plan;

/* Forward arguments.  Replaces FlashRNNFuncFused::forward(training, x, s0, R, b) -> {states, g_r, g_i}
 * (flashrnn/flashrnn/fused/flashrnn.cc:68-144); unlike the reference the tensors keep the user layouts, so the
 * permute + .contiguous() copies of flashrnn/flashrnn/flashrnn.py:1049-1057 disappear. */
typedef struct frnn_fwd_args {
  const void* Wx;      /* [B,T,Gw,N,D] dtype_io                      */
  const void* R;       /* [Gr,N,D,D]   dtype_io                      */
  const void* b;       /* [Gt,N,D]     dtype_io                      */
  const void* s0;      /* [S,B,1,N,D]  dtype_state                   */
  void* states;        /* [S,B,T,N,D]  dtype_state (output)          */
  void* cache;         /* cache_bytes, output; may be NULL when training == 0 or plan.cache_bytes == 0 */
  void* workspace;     /* workspace_bytes                            */
  void* last;          /* optional (NULL: off) [S,B,1,N,D] dtype_state (output): the states after step T-1 (one strided
                          device copy behind the time loop).  May be the very buffer `s0` points to: chunked or
                          token-by-token calls then carry their states in place                              */
  int64_t wx_stride[4]; /* element strides of the B, T, G, N dimensions of Wx (the D dimension is contiguous).  All
                           four 0: dense [B,T,Gw,N,D].  Each must be a non-negative multiple of 8 (16 bytes), else
                           FRNN_ERR_ALIGN                                                                          */
} frnn_fwd_args;

/* Backward arguments.  Replaces FlashRNNFuncFused::backward(R_t, b, s, g_r, g_i, ds_new) ->
 * {dWx, ds, dR, db} (flashrnn/flashrnn/fused/flashrnn.cc:146-246), including the post-loop cuBLAS dR GEMM and the
 * bias aggregation kernel (flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:1049-1069, 626-665).
 * dR || db are produced in fp32 inside the workspace (plan.grads_offset); frnn_finalize_grads casts them. */
typedef struct frnn_bwd_args {
  const void* R;        /* [Gr,N,D,D]  dtype_io                                      */
  const void* s0;       /* [S,B,1,N,D] dtype_state                                   */
  const void* states;   /* [S,B,T,N,D] dtype_state, as written by frnn_forward       */
  const void* cache;    /* as written by frnn_forward (training == 1); may be NULL when plan.cache_bytes == 0 */
  const void* dstates;  /* [S,B,T,N,D] dtype_state: cotangent of `states`            */
  void* dWx;            /* [B,T,Gw,N,D] dtype_io (output)                            */
  void* ds0;            /* [S,B,1,N,D] dtype_state (output)                          */
  void* workspace;      /* workspace_bytes; holds fp32 dR || db on return            */
  int64_t dstates_stride[4]; /* element strides of the S, B, T, N dimensions of dstates (D contiguous); all four 0:
                                dense [S,B,T,N,D]; multiples of 8 as for wx_stride                                 */
} frnn_bwd_args;

/* One word of device-side status per workspace: 0 = clean. */
typedef struct frnn_dev_status {
  uint32_t code;   /* 0 ok; 1 = a bounded device-side wait expired */
  uint32_t where;  /* kernel-specific location (time step)          */
  uint32_t cta;    /* linear CTA index that reported it            */
  uint32_t pad;
} frnn_dev_status;

/* ABI version of the loaded library (compare with FRNN_ABI_VERSION). */
int frnn_abi_version(void);

/* Pure host function: validates the problem and fills `out` (tile choice, cache/workspace sizes).
 * Replaces _FlashRNNCUDAFused.instance(config) (flashrnn/flashrnn/flashrnn.py:386-676): no JIT, no solver. */
int frnn_query(const frnn_problem* problem, frnn_plan* out);

/* Same as frnn_query but with the tile forced by the caller (used to measure the tile table);
 * any of the three may be 0 = "use the table's value".  Invalid combinations return FRNN_ERR_PLAN.
 * float32 problems: cluster_size 1..8 (units per CTA a multiple of 4, at most 64, its fp32 slice of R within shared
 * memory; cluster_size 1 otherwise selects the loops that stream R from L2), batch_tile 8, 4 or 2, wx_stages 0. */
int frnn_query_tile(const frnn_problem* problem, int cluster_size, int batch_tile, int wx_stages, frnn_plan* out);

/* Whole-sequence forward: one persistent launch (plus a small weight-repack launch).
 * Replaces ForwardPass::Run (flashrnn/flashrnn/fused/flashrnn_fused_forward.cu:772-975). */
int frnn_forward(const frnn_plan* plan, const frnn_fwd_args* args, void* stream);

/* Whole-sequence backward: reverse time loop + dR + db.  Replaces BackwardPass::Run
 * (flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:768-1086), without its host synchronisation. */
int frnn_backward(const frnn_plan* plan, const frnn_bwd_args* args, void* stream);

/* The two halves of frnn_backward, for callers that want to time or overlap them separately:
 * FRNN_PART_LOOP = zero the fp32 gradients, repack R^T, run the reverse time loop (dWx, ds0, db);
 * FRNN_PART_DR   = the dR reduction over all (b,t), which needs the loop's dWx.  frnn_backward = both, in order.
 * Same reference counterpart as frnn_backward (the reference also runs these as separate launches,
 * flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:947-1000 and 1049-1058). */
enum { FRNN_PART_LOOP = 1, FRNN_PART_DR = 2 };
int frnn_backward_parts(const frnn_plan* plan, const frnn_bwd_args* args, void* stream, int parts);

/* Forward pass WITHOUT a caller-provided workspace (args->workspace is ignored and may be NULL).
 * No counterpart in the reference.  Meant for callers that must not allocate device memory where they call the
 * library (a fixed arena handed out at start-up, a hot path on which cudaMalloc's device synchronisation is not
 * acceptable): the forward's scratch -- status block + R repacked into tensor-core fragments -- lives in a
 * file-scope device array of FRNN_NOALLOC_MAX_SCRATCH_BYTES inside the library, which every GPU that loads the
 * library holds until the process exits.  The entry point itself allocates and frees nothing, through the CUDA
 * runtime or any other library; what happens once per device is the driver loading this library's device code, see
 * "first call" below.
 *   - The plan is chosen as by frnn_query(problem).  Inputs, `states` and (training == 1) the activation `cache`
 *     of plan.cache_bytes (use frnn_query to size it) are still the caller's buffers.
 *   - Limit: 256 + Gr*N*D*D*2 bytes (float32 problems: *4; rounded up to 256) must fit FRNN_NOALLOC_MAX_SCRATCH_BYTES, else
 *     FRNN_ERR_TOO_LARGE is returned and nothing is launched.
 *   - First call on a device: it looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current).  If nothing of the library has run on that device yet, this lookup makes the driver load the
 *     library's device code, which is when the 8 MiB are set aside and which may synchronise the device.  Make that
 *     first call at start-up, before any stream capture and before the latency-critical phase.  To prime a device
 *     without launching work, call with a valid `problem` and an `args` whose tensor pointers are NULL: the address
 *     is looked up, then the call returns FRNN_ERR_NULL and nothing is enqueued.
 *   - All calls on one device share the array.  It keeps the previous call's contents; each call clears the status
 *     block and rewrites the fragments before use.  Two calls whose GPU work overlaps (different streams, or
 *     different host threads without ordering) race on it: order them on one stream or with events.
 *   - Launch errors come back through the return value.  The device-side status block of such a call sits in
 *     the internal array and cannot be read back; use frnn_forward with a workspace where that matters. */
#define FRNN_NOALLOC_MAX_SCRATCH_BYTES (8u << 20)
int frnn_forward_noalloc(const frnn_problem* problem, const frnn_fwd_args* args, void* stream);

/* Casts the fp32 gradients held in the workspace to dtype_io: dR[Gr,N,D,D], db[Gt,N,D].
 * `grads_f32` is workspace + plan->grads_offset (or a buffer of the same layout, e.g. after an all-reduce).
 * Replaces the reference's "accumulate in the parameter dtype" outputs (fused/flashrnn.cc:187-215). */
int frnn_finalize_grads(const frnn_plan* plan, const void* grads_f32, void* dR, void* db, void* stream);

/* Copies the device status word of a workspace to the host (synchronises `stream` first).
 * Replaces the int return + fprintf(stderr) error reporting of the reference's Run() functions
 * (flashrnn/flashrnn/fused/flashrnn_fused_forward.cu:935-969). */
int frnn_read_device_status(const void* workspace, void* stream, frnn_dev_status* out);

/* Human-readable text of a return code of this library (negative codes) or of CUDA (positive codes).
 * Replaces the TORCH_CHECK message strings of flashrnn/flashrnn/fused/flashrnn.cc:140-142, 238-240. */
const char* frnn_status_string(int code);

#ifdef __cplusplus
}
#endif
#endif /* FRNN_H_ */
