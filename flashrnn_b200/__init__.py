"""flashrnn_b200: B200-native (sm_100a) drop-in for the fused recurrent hot path of FlashRNN.

    from flashrnn_b200 import flashrnn, FlashRNNConfig
    states, last = flashrnn(Wx, R, b, states=None, function="lstm", backend="cuda_fused", dtype="bfloat16")
    stepper = FlashRNNStepper(R, b, function="lstm", batch_size=B); states_t = stepper.step(Wx_t)   # decoding
"""
from .flashrnn import FlashRNNConfig, flashrnn, _zero_state  # noqa: F401
from .stepper import FlashRNNStepper  # noqa: F401

__all__ = ["flashrnn", "FlashRNNConfig", "FlashRNNStepper"]
