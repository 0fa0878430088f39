"""qengine_b200: B200-native (sm_100a) operators for batch-1 speculative decoding of a hybrid
Gated-DeltaNet / gated-attention model with int4 group-128 weights.

Sub-modules: `_C` and `_w4` (operator surface over libqengine_b200.so), `quant` (W4 wire
format), `engine` (decode loop captured as CUDA graphs), `synth` (seeded synthetic models).
The CUDA library is required: importing `_C` / `_w4` fails if it has not been built
(`python -m qengine_b200.build`).
"""
__version__ = "0.1.0"
