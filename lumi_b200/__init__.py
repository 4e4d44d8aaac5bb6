"""lumi_b200 — B200 (sm_100a) implementation of lumi's token loop behind a C ABI.

`lumi_b200.api` mirrors the reference's `NmModel` / `generate`; `lumi_b200.synth` makes seeded
synthetic models in the reference's safetensors schema; `lumi_b200.build` compiles the CUDA library.
"""
from .api import NmModel, Session, Sampling, Stats, LumiError, TextCodec, generate, lib, LIB_PATH, EXPORTS  # noqa: F401
from .synth import ModelConfig  # noqa: F401
