"""Benchmark workloads: a GPT-2 shaped decoder (data-parallel training step) and a
Llama-3 shaped MLP / attention-output block (tensor-parallel step)."""
from .gpt2 import GPT2Config, GPT2Model  # noqa: F401
