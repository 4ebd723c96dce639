"""CPU oracle for the quantized DiT denoising step.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this directory; only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark do, and there only as the
checker or as the timed CPU arm, never as part of the GPU product path.

PARITY UNPINNED. The arithmetic restated here (mx.quantize, mx.quantized_matmul,
mx.fast.scaled_dot_product_attention, nn.LayerNorm / nn.RMSNorm / nn.gelu ...) lives in MLX, a
third-party dependency of the reference (pinned mlx==0.30.3 on linux / 0.31.0 on darwin in the
reference's pyproject.toml:69-70) whose source and wheel are not available offline. The
reference's own tests hold no packed weights, scales, biases or quantized-linear outputs. The
only reference golden vectors on this path are the LinearScheduler sigmas
(tests/schedulers/test_linear_scheduler.py:41-73), which `oracle.schedule` is pinned against.
"""
