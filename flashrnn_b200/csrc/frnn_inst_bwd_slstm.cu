// Instantiates the bwd time-loop kernel of the slstm cell for every supported head dim and batch tile.
#define FRNN_INST_CELL CELL_SLSTM
#define FRNN_INST_BWD 1
#define FRNN_INST_NAME get_bwd_kernel_slstm
#include "frnn_inst.cuh"
