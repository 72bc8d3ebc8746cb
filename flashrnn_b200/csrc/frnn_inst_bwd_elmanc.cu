// Instantiates the bwd time-loop kernel of the Elman cell with forward clamp (caches the tanh output).
#define FRNN_INST_CELL CELL_ELMAN_CLIP
#define FRNN_INST_BWD 1
#define FRNN_INST_NAME get_bwd_kernel_elmanc
#include "frnn_inst.cuh"
