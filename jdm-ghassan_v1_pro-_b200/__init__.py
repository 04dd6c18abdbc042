"""B200-native MoE decoder-LLM training and inference framework.

Layout: ``models`` (config, parameter table, CPU oracle and CUDA model), ``ops`` (Python launchers
for the sm_100a kernels in ``csrc/cuda``), ``parallel`` (peer-memory collectives, fused gradient
sync, expert parallelism, launcher), ``training`` (trainer, optimizers, scheduler, scaler,
checkpoints), ``inference`` (generator, KV cache, sampler, chat), ``formats`` (GGUF / GAI),
``data`` (tokenizer, shards, loaders, text pipeline), ``cli`` (entry points), ``utils``.
Native code: ``csrc/host`` (C++20, pybind11) and ``csrc/cuda`` (sm_100a kernels, C ABI).
"""
__version__ = "0.1.0"
