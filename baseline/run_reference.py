"""Reference arm of bench.py: drives the UNMODIFIED reference sources installed
under ``baseline/_ref`` through their own public functions
(``train.build_model`` / ``build_optimizer`` / ``all_reduce_grads`` / ``lr_at``
/ ``qk_clip`` / ``ema_update``, ``imf_video.IMFVideoLoss``) on the same
metric and config as ``bench.py``'s own arm.  None of this repository's
models, kernels or engine is on this path.

The reference's ``train.main()`` cannot be called directly for synthetic data:
its synthetic dataset branch raises a TypeError (it passes the (H, W) tuple
twice to ``torch.randn``), so the loop of ``main()`` is reproduced here call
for call with N(0,1) latents.  Attention: ``sdpa_flash`` (the reference's
``flash_jvp`` needs ``flash_attn.cute``, which is not installed), du/dt by its
Triton "fast" engine, bf16 autocast -- the configuration its authors ran on
A100.
"""

from __future__ import annotations

import copy
import json
import os
import sys
import time

MODEL_KW = {
    "d256": dict(hidden_size=256, depth=12, aux_head_depth=4, num_heads=4, kv_lora_rank=128),
    "d256_sla2": dict(hidden_size=256, depth=12, aux_head_depth=4, num_heads=4, kv_lora_rank=128,
                      attn_impl="sla2_cube_qat", sla2_tile=(4, 4, 4), sla2_topk=0.10),
    "d1024": dict(hidden_size=1024, depth=24, aux_head_depth=4, num_heads=16, kv_lora_rank=512,
                  max_params=600_000_000),
}
DATA_KW = {"d256": dict(latent_frames=20, latent_size=(56, 104)),
           "d256_sla2": dict(latent_frames=20, latent_size=(56, 104)),
           "d1024": dict(latent_frames=21, latent_size=(60, 104))}


def run(args, ref_dir, TOKENS, ClockSampler, L2Flush):
    if args.config not in MODEL_KW:
        raise RuntimeError(f"reference cannot run config {args.config!r} "
                           "(its kernels need head_dim 64 and power-of-two heads)")
    sys.path.insert(0, ref_dir)
    os.environ.setdefault("MOONLIGHT_COEFF_CACHE",
                          os.path.join(os.path.dirname(ref_dir), "ref_ns_coeffs.json"))
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise RuntimeError("reference arm needs a CUDA device (Triton kernels)")
    import config as rcfg_mod          # reference modules (top-level names)
    import train as rtrain
    from imf_video import IMFVideoLoss

    cfg = rcfg_mod.config
    for k, v in MODEL_KW[args.config].items():
        setattr(cfg.model, k, v)
    for k, v in DATA_KW[args.config].items():
        setattr(cfg.data, k, v)
    if "attn_impl" not in MODEL_KW[args.config]:
        cfg.model.attn_impl = "sdpa_flash"
    cfg.loss.jvp_impl = "fast"
    cfg.loss.autocast_bf16 = True
    cfg.optim.warmup_steps = 0

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device, backend = rtrain.resolve_device()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend)
    torch.manual_seed(cfg.run.seed + rank)

    net, _n, _attn = rtrain.build_model()
    net = net.to(device, dtype=getattr(torch, cfg.run.master_dtype))
    ema = copy.deepcopy(net).eval().requires_grad_(False)
    lc = cfg.loss
    loss_mod = IMFVideoLoss(
        net, cfg.model.num_classes, P_mean=lc.P_mean, P_std=lc.P_std,
        data_proportion=lc.data_proportion, cfg_beta=lc.cfg_beta,
        class_dropout_prob=lc.class_dropout_prob, jvp_impl=lc.jvp_impl,
        stratified_time=lc.stratified_time, stratified_interval=lc.stratified_interval,
        strat_group=0, s_max=lc.cfg_s_max, norm_p=lc.norm_p, norm_eps=lc.norm_eps,
        loss_v_weight=lc.loss_v_weight, autocast_bf16=lc.autocast_bf16)
    o = cfg.optim
    optimizer = rtrain.build_optimizer(net, o, device, verbose=False)
    params = list(net.parameters())

    B = cfg.data.batch_size_per_gpu
    h, w = cfg.data.latent_size
    shape = (B, cfg.model.in_channels, cfg.data.latent_frames, h, w)
    g = torch.Generator().manual_seed(1234 + rank)
    host_lat = [torch.randn(shape, generator=g).pin_memory() for _ in range(4)]
    host_lab = [torch.randint(0, cfg.model.num_classes, (B,), generator=g).pin_memory()
                for _ in range(4)]
    dev_lat = [t.to(device) for t in host_lat]
    dev_lab = [t.to(device) for t in host_lab]
    flush = L2Flush(device)

    def one_step(step, latents, labels, read_loss):
        optimizer.zero_grad(set_to_none=True)
        loss, parts = loss_mod(latents, labels)
        (loss / o.grad_accum).backward()
        val = loss.item() if read_loss else None
        if world > 1:
            rtrain.all_reduce_grads(params, world)
        lr = rtrain.lr_at(step)
        for grp in optimizer.param_groups:
            grp["lr"] = lr * grp.get("lr_width_mult", 1.0)
        gn = torch.nn.utils.clip_grad_norm_(net.parameters(), o.grad_clip)
        if torch.isfinite(gn):
            optimizer.step()
            rtrain.qk_clip(net, o.qk_clip_tau, world)
            rtrain.ema_update(ema, net, cfg.run.ema_decay)
        return val

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def max_ranks(x):
        if world > 1:
            t = torch.tensor([x], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return x

    for i in range(args.warmup):
        one_step(i, dev_lat[i % 4], dev_lab[i % 4], False)
    sync()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        flush()
        one_step(i, dev_lat[i % 4], dev_lab[i % 4], False)
    e1.record()
    sync()
    ms = max_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler is not None else None

    sync()
    t0 = time.perf_counter()
    last = None
    for i in range(args.steps):
        last = one_step(i, host_lat[i % 4].to(device, non_blocking=True),
                        host_lab[i % 4].to(device, non_blocking=True), True)
    sync()
    e2e_ms = max_ranks((time.perf_counter() - t0) * 1e3)

    tokens = TOKENS[args.config] * B * world
    if rank == 0:
        print(json.dumps({
            "impl": "reference",
            "metric": "latent tokens/sec/box per iMF train step (device-timed, max over ranks)",
            "value": tokens * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"model": f"reference IMFDiTVideo {args.config} attn={cfg.model.attn_impl} jvp=fast "
                                f"grad_checkpoint={cfg.model.grad_checkpoint}",
                       "global_batch": B * world, "seq_len": TOKENS[args.config],
                       "parallelism": f"dp{world} (flat fp32 NCCL all-reduce)"},
            "clocks": clocks,
            "e2e": {"value": tokens * args.steps / (e2e_ms / 1e3), "unit": "tokens/s",
                    "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": host_lat[0].numel() * 4 + host_lab[0].numel() * 8,
                    "d2h_bytes_per_step": 4, "loss": last},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()
