"""B200-native mixture-of-experts layer ops behind the reference's op signatures.

`ops` is the torch-tensor front end of the C ABI in include/b200_moe.h; `moe_layer.MoELayer` sequences the ops the
way the reference's transformer block does. The CUDA library must be built first
(`python -m ml_dataflow_b200.build`); nothing here falls back to PyTorch or the CPU.
"""
