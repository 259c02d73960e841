"""A single-GPU inference engine for NVIDIA B200 (sm_100a).

The package takes a model folder (``config.json`` + ``model.safetensors``) to
next-token logits and generated tokens.  It is built from replaceable parts:

``config``    typed configurations and the architecture registry
``weights``   safetensors reading/writing, binding by tensor name, random weights
``parts``     mixers, feed-forwards, norms, position encodings, block arrangements
``models``    architecture assemblies (one file per architecture)
``cache``     paged key/value cache manager with layer groups and state slots
``engine``    the step function, the scheduler and the entry points
``sampling``  greedy / temperature / top-k / top-p sampling
``csrc``      hand-written CUDA kernels for sm_100a and their build/loader

Importing the package never touches the GPU and never compiles anything;
kernels are compiled on first use (see ``csrc.build``).
"""

__version__ = "0.1.0"

from .config import load_config, register_architecture  # noqa: E402,F401
