"""Typed configuration tree for a training run.

The section and field names follow the TOML surface of the reference trainer
(reference: train/config.py:9-168) so an existing ``.toml`` keeps working:
``[model] [training] [data] [wandb]``.  Fields that the reference does not have
(expert parallelism, sequence-parallel norms, chunked cross-entropy, fp32 master
weights, synthetic data, fused NVLink collectives) are additions and all default
to values that reproduce the reference behaviour where one exists.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class ModelType(enum.Enum):
    """Model family; picked from ``model.model_name`` by substring
    (reference: train/train_qwen.py:121-128)."""

    QWEN3_5 = "qwen3_5"
    QWEN3_VL = "qwen3_vl"
    QWEN3_TEXT = "qwen3_text"

    @staticmethod
    def from_name(name: str) -> "ModelType":
        low = name.lower().replace("-", "").replace("_", "")
        if "qwen3.5" in low or "qwen35" in low:
            return ModelType.QWEN3_5
        if "vl" in low:
            return ModelType.QWEN3_VL
        if "qwen3" in low:
            return ModelType.QWEN3_TEXT
        raise ValueError(f"cannot infer the model family from model_name={name!r}")


@dataclass
class ModelSection:
    model_name: str = "NULL"
    # kept for TOML compatibility; only the native implementation exists here
    model_impl: str = "native"
    train_llm: bool = True
    train_mlp: bool = True
    train_vit: bool = False
    # --- additions ---
    # architecture preset used when there is no snapshot directory
    # ("tiny-qwen3", "qwen3-8b", "qwen3-vl-8b", "qwen3.5-dense", "qwen3.5-moe", ...)
    preset: str = ""
    # DSA sparse attention on the full-attention layers (Qwen3.5 only)
    dsa: bool = False
    dsa_topk: int = 2048


@dataclass
class WandbSection:
    run_name: str = "default"
    project_name: str = "vlm_training_b200"
    entity_name: str = ""
    log_topk: bool = True
    top_k: int = 4
    # addition: "online" | "offline" | "disabled"
    mode: str = "disabled"


@dataclass
class TrainingSection:
    model_dir: str = "NULL"
    output_dir: str = "checkpoints"
    load_text_model: bool = False
    text_model_dir: str = "NULL"
    load_vision_model: bool = False
    vision_model_dir: str = "NULL"
    resume_checkpoint: bool = False
    save_steps: int = 1000
    bfloat16: bool = True
    lr_llm: float = 2e-6
    lr_mlp: float = 1e-5
    lr_vit: float = 1e-6
    random_init: bool = False
    tpi_multiplier: float = 1.0
    eps: float = 1e-8
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    scheduler_type: str = "wsd"
    total_steps: int = 1000
    warmup_steps: int = 50
    wsd_decay_ratio: float = 0.1
    min_lr_ratio: float = 0.1
    data_parallel: str = "ddp"  # "fsdp" | "ddp"
    tp_size: int = 1
    async_tp: bool = True
    compile: bool = True  # accepted and ignored: there is no tracing compiler here
    ac_mode: str = "off"  # "off" | "full" | "sac"
    # --- additions ---
    ep_size: int = 1
    sequence_parallel: bool = False
    ce_chunk_size: int = 1024
    fp32_master: bool = True
    # storage type of the Adam moments ("fp32" | "bf16"); master weights stay fp32 either way
    optimizer_state_dtype: str = "fp32"
    # gradient clipping is off unless asked for: the reference never clips
    # although it carries max_grad_norm (reference: train/train_qwen.py:534-605)
    clip_grad: bool = False
    # one-kernel NVLink paths (reduce-scatter+AdamW+all-gather, TP GEMM+collective)
    fused_comm: bool = True
    # with data_parallel = "fsdp": also shard the bf16 parameters and gradients over the data-parallel ranks (ZeRO-3:
    # a layer's parameters are gathered for its forward / backward and released afterwards).  Off: parameters and
    # gradients stay whole on every rank and only the optimizer state is sharded, which is faster while the model fits.
    reshard_params: bool = False
    # release a unit's gathered parameters right after its forward pass (and gather again for backward);
    # false keeps them until the unit's backward pass is done (the reference's default FSDP policy)
    reshard_after_forward: bool = True
    # with reshard_params on GPUs (fused_comm, no tensor parallelism): a block's first weight (qkv / in_proj) is gathered by
    # the GEMM that reads it instead of by the block's parameter gather
    reshard_fuse_first_gemm: bool = True
    # FP8 GEMMs (tensor-wise dynamic scaling; e4m3 forward, e5m2 output gradients) for the language model's linear layers
    # whose dimensions are multiples of 16; the vision tower, the LM head and MoE experts stay bf16
    float8: bool = False
    beta1: float = 0.9
    beta2: float = 0.999
    seed: int = 42
    backend: str = "auto"  # "auto" | "nccl" | "gloo"
    device: str = "auto"  # "auto" | "cuda" | "cpu"
    log_every: int = 1
    # on a GPU, read a step's loss / reductions / device status one step later from pinned memory instead of
    # stalling the host on them (metrics of step k are returned by the call that runs step k + 1)
    async_metrics: bool = True
    # "DEBUG" runs: first and last optimizer step of the cProfile window (reference: train/train_qwen.py:667-694)
    cprofile_start: int = 50
    cprofile_stop: int = 65


@dataclass
class DataSection:
    data_path: str = "NULL"
    shuffle_buffer_size: int = 100
    max_samples_per_sequence: int = 100
    packing_buffer_size: int = 0
    batch_size: int = 4
    text_dataset: bool = False
    seq_len: float = 4096
    # --- additions ---
    # "" (real data through the energon adapter) or a synthetic generator name:
    # "text-uniform", "text-loguniform", "vlm"
    synthetic: str = ""
    doc_len_min: int = 128
    doc_len_max: int = 8192
    num_workers: int = 2
    # rows are produced by this many worker processes per rank (0: by one thread of the training process); a worker reads its
    # own 1/n of the rank's samples, the training process takes the workers' rows in round-robin order
    worker_processes: int = 0
    # cooker for crude webdataset samples: "auto" (from the sample's fields) or a name of data.cookers.COOKERS
    cooker: str = "auto"


@dataclass
class Config:
    training: TrainingSection = field(default_factory=TrainingSection)
    model: ModelSection = field(default_factory=ModelSection)
    data: DataSection = field(default_factory=DataSection)
    wandb: WandbSection = field(default_factory=WandbSection)
    # present only so ``--config path`` is itself a recognised option
    config: str = ""
