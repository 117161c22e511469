"""Native backend of the quantized-linear path: the `fp4t` C-ABI library (hand-written
sm_100a CUDA) and the `torch.ops.xops` operator registrations built on it."""
