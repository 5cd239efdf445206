"""Configuration tree for iMF video training on B200.

Same field names and groups as the reference's module-level dataclass tree
(reference ``config.py:11-223``) so a reference user finds every knob where
they expect it, plus three things the reference lacks: dict / dotted-key
overrides (``apply_overrides``), a CLI/YAML front end (``parse_cli``) and a
``parallel`` group for the NVLink-side knobs that only exist here.
"""

from __future__ import annotations

import ast
import copy
import dataclasses
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, Optional


@dataclass
class ModelConfig:
    hidden_size: int = 1024
    depth: int = 19                 # shared blocks = depth - aux_head_depth
    aux_head_depth: int = 4         # blocks in each of the u and v branches
    num_heads: int = 16
    # MLA geometry; 0 means "derive from head_dim / hidden_size"
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    patch_size: tuple = (1, 2, 2)
    in_channels: int = 16
    num_classes: int = 1000
    # "flash_jvp" | "sla2_jvp" | "sla2_cube_qat" | "sdpa_flash" | "sdpa"
    attn_impl: str = "flash_jvp"
    mla_use_output_gate: bool = True
    # SLA2 sparse-linear attention
    sla2_topk: float = 0.03
    sla2_bq: int = 128
    sla2_bk: int = 64
    sla2_alpha_init: float = 0.9
    sla2_tile: tuple = (4, 4, 4)
    mlp_ratio: float = 8 / 3
    situ_beta: float = 4.0
    situ_linear_beta: Optional[float] = 25.0
    rmsnorm_eps: float = 1e-5
    num_class_tokens: int = 8
    num_time_tokens: int = 4
    num_cfg_tokens: int = 4
    num_interval_tokens: int = 2
    freq_embedding_size: int = 256
    token_init_constant: float = 1.0
    embedding_init_constant: float = 1.0
    weight_init_constant: float = 0.5
    rope_theta: float = 10000.0
    attn_res_block_size: int = 4
    grad_checkpoint: bool = True
    eval_mode: bool = False
    max_params: int = 300_000_000


@dataclass
class DataConfig:
    batch_size_per_gpu: int = 1
    latent_dir: str = ".cache/wan_syn_2k_full"   # or "synthetic"
    latent_frames: int = 20
    latent_size: tuple = (56, 104)
    num_workers: int = max(0, (os.cpu_count() or 1) - 2)
    pin_memory: bool = True


@dataclass
class LossConfig:
    P_mean: float = -0.4
    P_std: float = 1.0
    data_proportion: float = 0.25
    cfg_beta: float = 1.0
    cfg_s_max: float = 7.0
    class_dropout_prob: float = 0.1
    norm_p: float = 1.0
    norm_eps: float = 0.01
    loss_v_weight: float = 1.0
    # "fused": one dual-number pass gives u, du/dt and v (this framework's
    # production path); "fast": alias of "fused" kept for reference configs;
    # "functorch": torch.func.jvp over the plain forward (oracle path).
    jvp_impl: str = "fast"
    autocast_bf16: bool = False
    stratified_time: bool = True
    stratified_interval: bool = False
    strat_group_auto: bool = False


@dataclass
class OptimConfig:
    optimizer: str = "moonlight"
    lr: float = 2e-3
    weight_decay: float = 0.1
    betas: tuple = (0.9, 0.95)
    muon_momentum: float = 0.9
    muon_nesterov: bool = True
    muon_ns_steps: int = 5
    muon_lr_scale_constant: float = 0.2
    muon_coeff_mode: str = "per_shape"
    muon_coeff_samples: int = 32
    muon_coeff_iters: int = 3000
    muon_coeff_lr: float = 2e-2
    muon_coeff_seed: int = 0
    grad_clip: float = 1.0
    qk_clip_tau: float = 40.0
    lr_schedule: str = "wsd"
    warmup_steps: int = 100
    total_steps: int = 4000
    decay_fraction: float = 0.2
    decay_shape: str = "1-sqrt"
    min_lr_ratio: float = 0.1
    grad_accum: int = 1
    fused_adamw: bool = True
    ns_cuda_graph: bool = False      # replay the Newton-Schulz phase of the optimizer as one CUDA graph


@dataclass
class RunConfig:
    seed: int = 0
    out_dir: str = "checkpoints"
    log_every: int = 50
    ckpt_every: int = 5000
    resume: str = ""
    ema_decay: float = 0.9999
    wandb_project: str = ""
    master_dtype: str = "float32"
    # extras (not in the reference): phase timers / NVTX ranges, heartbeat
    profile_phases: bool = False
    # the host waits for loss / norm / skip flag only (copied out before the update kernels) and
    # reports QK-clip statistics and the kernel status word one step late
    overlap_stats_read: bool = True
    # fixed-order dQ accumulation in the attention backward: training steps become bit-identical
    # from run to run (costs 13-34 % of that kernel's time)
    deterministic: bool = False
    heartbeat_s: float = 0.0


@dataclass
class SampleConfig:
    num_steps: int = 1
    omega: float = 2.0
    t_min: float = 0.0
    t_max: float = 1.0


@dataclass
class ParallelConfig:
    """NVLink-side knobs; no counterpart in the reference (it only has a flat
    NCCL all-reduce, reference ``train.py:353-371``)."""

    # "fused_p2p": own reduce-scatter/all-gather kernels over peer memory;
    # "nccl_flat": the reference's single flat all-reduce; "nccl_bucketed".
    grad_sync: str = "fused_p2p"
    bucket_mb: float = 32.0
    # give every Muon matrix one owner rank; the others receive the update
    distributed_moonlight: bool = True
    # what the peers' gradient contributions travel as ("bfloat16": bucketed reduce with fp32
    # accumulation and sharded AdamW; "float32": one whole-arena fp32 reduce after backward)
    wire_dtype: str = "bfloat16"
    # launch each block's gradient bucket on a side stream as soon as backward has produced it
    overlap_backward: bool = True
    broadcast_init: bool = True
    # bound (seconds) of every device-side wait on another rank's flag; when it runs out the
    # kernel returns without touching data and the trainer raises at its per-step host read
    peer_wait_s: float = 2.0


@dataclass
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    data: DataConfig = field(default_factory=DataConfig)
    loss: LossConfig = field(default_factory=LossConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    run: RunConfig = field(default_factory=RunConfig)
    sample: SampleConfig = field(default_factory=SampleConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)


config = Config()


def config_as_dict(cfg: Optional[Config] = None) -> Dict[str, Any]:
    """Plain nested dicts (safe for ``torch.load(weights_only=True)``);
    reference ``train.py:33-41``."""
    return dataclasses.asdict(config if cfg is None else cfg)


def _coerce(old: Any, new: Any) -> Any:
    if isinstance(new, str) and not isinstance(old, str):
        try:
            new = ast.literal_eval(new)
        except (ValueError, SyntaxError):
            if isinstance(old, bool):
                new = new.lower() in ("1", "true", "yes", "on")
    if isinstance(old, tuple) and isinstance(new, list):
        new = tuple(new)
    if isinstance(old, bool) and not isinstance(new, bool):
        new = bool(new)
    elif isinstance(old, float) and isinstance(new, int) and not isinstance(new, bool):
        new = float(new)
    return new


def apply_overrides(cfg: Config, overrides: Dict[str, Any]) -> Config:
    """Apply ``{"model.hidden_size": 256, "optim": {"lr": 1e-3}}`` style
    overrides in place. Unknown keys raise ``KeyError`` (typos must not pass
    silently)."""
    for key, value in overrides.items():
        if isinstance(value, dict):
            apply_overrides(cfg, {f"{key}.{k}": v for k, v in value.items()})
            continue
        obj = cfg
        parts = key.split(".")
        for p in parts[:-1]:
            if not hasattr(obj, p):
                raise KeyError(f"unknown config group {p!r} in {key!r}")
            obj = getattr(obj, p)
        leaf = parts[-1]
        if not hasattr(obj, leaf):
            raise KeyError(f"unknown config key {key!r}")
        setattr(obj, leaf, _coerce(getattr(obj, leaf), value))
    return cfg


def load_config_dict(cfg: Config, tree: Dict[str, Any]) -> Config:
    """Restore a ``config_as_dict`` tree (e.g. from a checkpoint); keys that
    this build does not know are ignored so older checkpoints still load."""
    for group, values in tree.items():
        if not hasattr(cfg, group) or not isinstance(values, dict):
            continue
        g = getattr(cfg, group)
        for k, v in values.items():
            if hasattr(g, k):
                setattr(g, k, _coerce(getattr(g, k), v))
    return cfg


def parse_cli(argv: Iterable[str], cfg: Optional[Config] = None) -> Config:
    """``--config file.yaml``, ``--preset name`` and/or ``group.key=value`` tokens."""
    cfg = config if cfg is None else cfg
    argv = list(argv)
    i = 0
    while i < len(argv):
        tok = argv[i]
        if tok == "--config":
            import yaml

            with open(argv[i + 1]) as fh:
                apply_overrides(cfg, yaml.safe_load(fh) or {})
            i += 2
            continue
        if tok == "--preset":
            load_config_dict(cfg, config_as_dict(preset(argv[i + 1])))
            i += 2
            continue
        if "=" not in tok:
            raise SystemExit(f"expected group.key=value, got {tok!r}")
        k, v = tok.lstrip("-").split("=", 1)
        apply_overrides(cfg, {k: v})
        i += 1
    return cfg


def preset(name: str) -> Config:
    """Named configurations used by the benchmarks and tests.

    ``tiny``   d=64, 3 blocks, 276 tokens (CPU plumbing).
    ``d256``   d=256, depth 12, 4 heads, 29,140 tokens (headline benchmark).
    ``d256_sla2``  same with cube SLA2 INT8-QAT attention.
    ``d1024``  d=1024, depth 24, 16 heads, 32,780 tokens.
    ``wan1p3b`` d=1536, 30 layers, 12 heads (head_dim 128), FFN 8960, SLA2 cube attention.
    ``wan1p3b_dense`` the same geometry with dense attention (the fused primal+tangent
    kernels cover head_dim 128 for dense attention).
    """
    c = copy.deepcopy(Config())
    m, d = c.model, c.data
    d.latent_dir = "synthetic"
    if name == "tiny":
        m.hidden_size, m.depth, m.aux_head_depth, m.num_heads = 64, 2, 1, 2
        m.kv_lora_rank, m.qk_rope_head_dim = 32, 16
        m.mlp_ratio = 4.0
        m.attn_impl = "sdpa"
        m.attn_res_block_size = 0
        m.grad_checkpoint = False
        d.batch_size_per_gpu, d.latent_frames, d.latent_size = 2, 4, (16, 16)
    elif name in ("d256", "d256_sla2"):
        m.hidden_size, m.depth, m.aux_head_depth, m.num_heads = 256, 12, 4, 4
        m.kv_lora_rank = 128
        m.grad_checkpoint = False
        d.latent_frames, d.latent_size = 20, (56, 104)
        c.loss.autocast_bf16 = True
        if name == "d256_sla2":
            m.attn_impl = "sla2_cube_qat"
            m.sla2_topk = 0.10
    elif name == "d1024":
        m.hidden_size, m.depth, m.aux_head_depth, m.num_heads = 1024, 24, 4, 16
        m.kv_lora_rank = 512
        m.max_params = 600_000_000
        m.grad_checkpoint = False          # activations of all 28 blocks fit in 180 GB
        d.latent_frames, d.latent_size = 21, (60, 104)
        c.loss.autocast_bf16 = True
    elif name in ("wan1p3b", "wan1p3b_dense"):
        m.hidden_size, m.depth, m.aux_head_depth, m.num_heads = 1536, 30, 4, 12
        m.mlp_ratio = 8960 / 1536
        if name == "wan1p3b":
            m.attn_impl = "sla2_cube_qat"
            m.sla2_topk = 0.10
        m.max_params = 2_000_000_000
        # 34 blocks x 32,780 rows x ~106 KB of saved activations per row would leave no room
        # beside 1.7 B parameters with their optimizer state: recompute each block in backward
        m.grad_checkpoint = True
        d.latent_frames, d.latent_size = 21, (60, 104)
        c.loss.autocast_bf16 = True
    else:
        raise KeyError(f"unknown preset {name!r}")
    return c
