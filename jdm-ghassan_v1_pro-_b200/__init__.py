"""B200-native MoE decoder-LLM training and inference framework.

Layout: ``models`` (config, parameter table, CPU oracle and CUDA model), ``ops`` (Python launchers
for the sm_100a kernels in ``csrc/cuda``), ``parallel`` (peer-memory collectives, fused gradient
sync, expert parallelism, launcher), ``training`` (trainer, optimizers, scheduler, scaler,
checkpoints), ``inference`` (generator, KV cache, sampler, chat), ``formats`` (GGUF / GAI),
``data`` (tokenizer, shards, loaders, text pipeline), ``cli`` (entry points), ``utils``.
Native code: ``csrc/host`` (C++20, pybind11) and ``csrc/cuda`` (sm_100a kernels, C ABI).
"""
__version__ = "0.1.0"


def _use_alternate_host_library():
    """``GB200_HOST_SO=<file>`` loads the host extension from that file instead of the one beside this package: a
    sanitizer-instrumented build (``python -m ghassan_b200.build --sanitize address|thread``)."""
    import os
    import sys
    path = os.environ.get("GB200_HOST_SO", "")
    if not path:
        return
    import importlib.machinery
    import importlib.util
    name = __name__ + "._gb200_host"
    loader = importlib.machinery.ExtensionFileLoader(name, path)
    spec = importlib.util.spec_from_file_location(name, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[name] = mod
    globals()["_gb200_host"] = mod


_use_alternate_host_library()
