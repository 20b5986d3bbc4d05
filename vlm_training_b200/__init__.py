"""vlm_training_b200 — a Blackwell-native (sm_100a) VLM pre-training framework.

Sub-packages
------------
config    TOML / CLI configuration tree
models    Qwen3, Qwen3-VL and Qwen3.5 (dense + MoE) with HF state-dict key layout
ops       functional hot ops: CUDA (sm_100a) implementations with torch oracles
parallel  device mesh, sharded data parallel, tensor / expert parallel, peer memory
data      synthetic generators, sequence packing, task encoders
train     trainer, optimizer, schedulers, checkpointing, metrics
utils     checkpoint conversion, chat, snapshot download, misc helpers
eval      perplexity evaluation
"""

__version__ = "0.1.0"
