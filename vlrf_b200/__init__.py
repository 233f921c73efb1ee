"""vlrf_b200: a small, whole GPT-2 inference library for one NVIDIA B200 (sm_100a).

config/    typed configurations from config.json, presets as data
registry   architecture name → configuration class, tensor list, random weights, builder
weights/   safetensors by tensor name, the one error that lists every mismatch, random-weights mode
parts/     norm, position encoding, mixer (attention), feed-forward, block; chosen layer by layer
cache/     slots and blocks per sequence, groups of layers with storage of their own, fixed-size state
engine/    the model as data, the step function, the generation loop
sampling/  options, the per-request random stream, the device sampler
csrc/      the CUDA kernels and their loader
"""
from .api import Model
from .sampling.params import SamplingParams

__version__ = "0.1.0"
__all__ = ["Model", "SamplingParams", "__version__"]
