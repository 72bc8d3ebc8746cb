// Instantiates the fwd time-loop kernel of the Elman cell with forward clamp (caches the tanh output).
#define FRNN_INST_CELL CELL_ELMAN_CLIP
#define FRNN_INST_BWD 0
#define FRNN_INST_NAME get_fwd_kernel_elmanc
#include "frnn_inst.cuh"
