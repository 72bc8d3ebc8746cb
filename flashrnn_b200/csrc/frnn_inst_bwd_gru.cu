// Instantiates the bwd time-loop kernel of the gru cell for every supported head dim and batch tile.
#define FRNN_INST_CELL CELL_GRU
#define FRNN_INST_BWD 1
#define FRNN_INST_NAME get_bwd_kernel_gru
#include "frnn_inst.cuh"
