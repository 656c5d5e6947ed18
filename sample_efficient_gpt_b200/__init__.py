"""B200-native sample-efficient GPT pretraining framework.

Layers, bottom-up: ``csrc`` (sm_100a CUDA kernels) -> ``ops`` (autograd functions that
dispatch to the CUDA extension on a GPU and to a plain PyTorch restatement on CPU) ->
``models`` -> ``optim`` -> ``parallel`` -> ``training`` -> ``train.py`` CLI.
"""

__version__ = "0.1.0"
