"""coccl_b200: a Blackwell-native compression-aware collective framework.

Layers (top to bottom): models/ (GPT, MoE), parallel/ (DP/ZeRO-1, TP+SP, PP, EP,
communicator + process-group backend), ops/ (kernel front ends), csrc/ (C++17
host runtime: TOML policy model, router, planner, autotuner, training
classifier, plugin SDK, symmetric memory; and the sm_100a kernels).
"""
__version__ = "0.1.0"
