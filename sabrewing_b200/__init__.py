"""B200-native MoE-block hot path behind the sabrewing C descriptor / lag_cuda_* C-ABI."""
