// Instantiates the fwd time-loop kernel of the elman cell for every supported head dim and batch tile.
#define FRNN_INST_CELL CELL_ELMAN
#define FRNN_INST_BWD 0
#define FRNN_INST_NAME get_fwd_kernel_elman
#include "frnn_inst.cuh"
