"""CPU oracle for the FlashRNN recurrent hot path.  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this package;
the shipped CUDA path never does.  Two restatements live here:

* ``oracle.c_oracle`` -- ctypes front end of ``frnn_oracle.c`` (plain C, fp64 and fp32, forward and
  closed-form backward; OpenMP over independent batch rows and heads).
* ``oracle.vanilla_port`` -- a PyTorch restatement of the reference's ``vanilla`` CPU backend (the loop
  over time with autograd providing the backward); used as the timed CPU baseline and as a second,
  independent check of the C code.
"""
from .c_oracle import CELLS, build_oracle, oracle_forward, oracle_fwbw, cell_dims  # noqa: F401
