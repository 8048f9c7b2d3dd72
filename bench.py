#!/usr/bin/env python
"""Flash-MVPA forward benchmark (one JSON line on rank 0).

Workload: BASELINE config 2 per GPU — bf16 forward, batch 4, 64 channels x 64 time segments
(4096 tokens), 16 heads (MHA), head_dim 64, window 10; Q/K/V, relative keys and biases ~ N(0,1),
seed 1.  With N GPUs every rank runs that workload on its own batch shard (weak scaling, no
data-path collective: batch elements are independent).

  value     whole-job TFLOP/s with inputs resident in HBM, counted with the window-aware
            algorithmic flop count F_alg = 2D(P_c+P_w) + 2DN(T+C) per (batch, head)
  e2e       same metric through `attentions.flashmvpa` with HOST buffers: pinned host->device
            copies of q/k/v and the device->host read of o are inside the timed region
  roofline  dominant kernel vs the measured dense bf16 peak (MEASURED_PEAKS.json, burst figure)
  cpu_baseline  the materialised PyTorch attention (oracle/mvpa_port_torch.py, a port of the
            reference's `_rel_attn`) on the host cores, on a bounded sample of the same workload
  extra     model_cfg4 / model_cfg5: full-model forward tokens/s on synthetic iEEG, the batch split over the
            ranks; long_sample_16k (N >= 2): one 16k-token sample with its time axis spread over the ranks and
            the K/V all-gather overlapped; the 16k-token and config-3 operator points, forward and forward +
            backward; triton_reference: the reference's own Triton operator on the same GPU; cpu_config1:
            BASELINE config 1 on the host cores

`--impl reference` times only that CPU port (rank 0), as the reference arm; `--impl triton` runs the
reference's Triton operator staged under baseline/_ref/ (what `extra.triton_reference` calls in a child process).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "multi-variate-parallel-transformer_b200"))

WORKLOADS = {
    # BASELINE config 2: the configuration the headline metric is quoted on
    "cfg2": (dict(B=4, H=16, Hkv=16, T=64, C=64, D=64, window=10),
             "cfg2: bf16 fwd, B4 x 16 heads (MHA) x 4096 tokens (64 ch x 64 seg), head_dim 64, window 10"),
    # forward half of BASELINE config 3
    "cfg3": (dict(B=8, H=16, Hkv=16, T=128, C=32, D=64, window=10),
             "cfg3 fwd: bf16, B8 x 16 heads (MHA) x 4096 tokens (32 ch x 128 seg), head_dim 64, window 10"),
    # one sample-layer of BASELINE config 5 (the 16k-token target of the north star)
    "16k": (dict(B=1, H=16, Hkv=8, T=128, C=128, D=128, window=10),
            "16k tokens: bf16 fwd, B1 x 16 heads / 8 kv heads x 16384 tokens (128 ch x 128 seg), head_dim 128"),
    # one layer of BASELINE config 5 at its full batch (4.3 GB of q, k, v per step)
    "cfg5": (dict(B=32, H=16, Hkv=8, T=128, C=128, D=128, window=10),
             "cfg5 layer: bf16 fwd, B32 x 16 heads / 8 kv heads x 16384 tokens (128 ch x 128 seg), head_dim 128"),
}
WORKLOAD, NAME = WORKLOADS["cfg2"]
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the forward kernel, from the ncu
# captures summarised under profiles/ (bytes)
NCU_DRAM_BYTES = {"cfg2": 137.2e6, "16k": 208.2e6}
METRIC = "flash_mvpa_fwd_tflops"
UNIT = "TFLOP/s (F_alg)"


def flops(B, H, T, C, D, window=10, **_):
    N = T * C
    p_c = C * C * T * (T + 1) // 2
    p_w = C * C * (sum(min(t, window) + 1 for t in range(T - 1)) + T)
    return dict(f_alg=B * H * (2 * D * (p_c + p_w) + 2 * D * N * (T + C)), f_dense=B * H * 4 * D * p_c)


def flops_bwd(B, H, T, C, D, window=10, **_):
    """Algorithmic backward count: dV, dP over causal pairs; recomputed S, dQ, dK over windowed pairs;
    recomputed relative scores and their two gradient products each."""
    N = T * C
    p_c = C * C * T * (T + 1) // 2
    p_w = C * C * (sum(min(t, window) + 1 for t in range(T - 1)) + T)
    return B * H * (2 * D * (2 * p_c + 3 * p_w) + 6 * D * N * (T + C))


def peaks(sustained=False):
    """Burst figure for kernels of under a millisecond timed alone; the sustained one for steps of tens of
    milliseconds, which run under the power cap (the config-5 workload)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        if sustained:
            return float(m["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
        return float(m["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        if sustained:
            return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier pool measurement)"
        return 1590.0, "fallback (1.59 PFLOP/s, earlier pool measurement)"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs (a thread
    in this process, every 2 ms); falls back to one `nvidia-smi` query if NVML is missing."""

    def __init__(self, index):
        self.index, self.rows, self.stop, self.thread, self.max_mhz = index, [], False, None, None

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            masks = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                     "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                     "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}

            def loop():
                while not self.stop:
                    try:
                        mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                        try:
                            r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                        except Exception:
                            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                        self.rows.append((float(mhz), [n for n, m in masks.items() if r & m]))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x for x in vis.split(",") if x.strip() != ""]
            if self.index < len(ids) and ids[self.index].strip().isdigit():
                return int(ids[self.index])
        return self.index

    def __exit__(self, *a):
        self.stop = True
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.rows:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True).stdout
                a, b = (float(x) for x in out.strip().split(","))
                return {"sm_mhz": a, "sm_max_mhz": b, "reasons": [], "samples": 0, "note": "idle nvidia-smi query"}
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [r[0] for r in self.rows]
        reasons = sorted({n for r in self.rows for n in r[1]})
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(sm)}


def use_all_host_threads(torch):
    """`torch.distributed.run` exports OMP_NUM_THREADS=1 to its workers; the CPU legs use every core the
    process may run on, whatever launched them, so that `cores` is the same at every GPU count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


_REF_LAYER = None


def reference_layer_class():
    """The reference's own `MVPFormerGQAAttention` (`layers/mvpa.py`), loaded unmodified from baseline/_ref/
    where the build staged it, or None when it is not there.  Only its CPU method `_rel_attn` is used; the
    `loralib` import it makes (for LoRA fine-tuning, off here) is answered with an empty module."""
    global _REF_LAYER
    if _REF_LAYER is None:
        _REF_LAYER = False
        ref = os.path.join(ROOT, "baseline", "_ref")
        if os.path.exists(os.path.join(ref, "layers", "mvpa.py")) and os.path.exists(os.path.join(ref, "attentions")):
            import importlib
            import types
            mine = lambda k: k in ("attentions", "layers", "loralib") or k.startswith(("attentions.", "layers."))
            saved_path, saved_mods = list(sys.path), {k: m for k, m in sys.modules.items() if mine(k)}
            try:
                for k in saved_mods:
                    del sys.modules[k]
                sys.modules["loralib"] = types.ModuleType("loralib")
                sys.path.insert(0, ref)
                _REF_LAYER = importlib.import_module("layers.mvpa").MVPFormerGQAAttention
            except Exception:
                _REF_LAYER = False
            finally:   # this library's own `attentions` / `layers` stay what the rest of the bench imports
                sys.path[:] = saved_path
                for k in [k for k in sys.modules if mine(k)]:
                    del sys.modules[k]
                sys.modules.update(saved_mods)
    return _REF_LAYER or None


def cpu_attention(sample, seed):
    """(callable running one pass of the materialised attention over `sample`, kind): the reference's own
    `_rel_attn` when baseline/_ref/ holds it ("reference"), else its port in oracle/ ("port")."""
    import torch
    B, H, Hkv, T, C, D = (sample[k] for k in ("B", "H", "Hkv", "T", "C", "D"))
    g = torch.Generator().manual_seed(seed)
    N = T * C
    r = lambda *s: torch.randn(*s, generator=g)
    q, u, vt, z, k, rt, rc, v = (r(B, H, N, D), r(Hkv, D), r(Hkv, D), r(Hkv, D), r(B, Hkv, N, D), r(Hkv, T, D),
                                 r(Hkv, C, D), r(B, Hkv, N, D))
    cls = reference_layer_class()
    if cls is not None:
        from types import SimpleNamespace as NS
        cfg = NS(max_position_embeddings=T, hidden_size=H * D, num_attention_heads=H, n_head_kv=Hkv, n_inner=4 * H * D,
                 global_att=True, scale_attn_weights=True, scale_attn_by_inverse_layer_idx=False,
                 reorder_and_upcast_attn=False, lora=False, attn_pdrop=0.0, resid_pdrop=0.0)
        layer = cls(cfg, layer_idx=0).eval()
        layer.attn_bias.data = torch.cat([u.flatten(), vt.flatten(), z.flatten()])
        a = (q.view(B, H, T, C, D), k.view(B, Hkv, T, C, D), rt.view(1, Hkv, T, 1, D), rc.view(1, Hkv, 1, C, D),
             v.view(B, Hkv, T, C, D))
        return (lambda: layer._rel_attn(*a)), "reference"
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import mvpa_port_torch as port
    return (lambda: port.rel_attn(q, u, vt, z, k, rt, rc, v, D ** -0.5, sample["window"])), "port"


def cpu_port_time(sample, reps=1, seed=1):
    """(seconds per pass of the materialised PyTorch attention over `sample` on the host cores, threads, kind)."""
    import torch
    use_all_host_threads(torch)
    fn, kind = cpu_attention(sample, seed)
    ts = []
    with torch.no_grad():
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
    return statistics.median(ts), torch.get_num_threads(), kind


def cpu_config1():
    """BASELINE config 1 exactly: the materialised attention (`layers/mvpa.py:173-278`, here its port) at
    batch 1, 16 channels x 32 segments, 4 heads, head_dim 64, fp32, seed 0, on the host cores:
    3 warm-up passes, 20 timed."""
    import torch
    threads = use_all_host_threads(torch)
    B, H, Hkv, T, C, D = 1, 4, 4, 32, 16, 64
    fn, kind = cpu_attention(dict(B=B, H=H, Hkv=Hkv, T=T, C=C, D=D, window=10), seed=0)
    ts = []
    with torch.no_grad():
        for i in range(23):
            t0 = time.perf_counter()
            fn()
            if i >= 3:
                ts.append(time.perf_counter() - t0)
    f = flops(B, H, T, C, D)["f_alg"]
    return {"workload": "config 1: fp32, B1 x 4 heads x 512 tokens (16 ch x 32 seg), head_dim 64", "reps": len(ts),
            "kind": kind,
            "mean_ms": 1e3 * statistics.mean(ts), "median_ms": 1e3 * statistics.median(ts),
            "tflops_f_alg": f / statistics.median(ts) / 1e12, "torch_threads": threads, "cpu_count": os.cpu_count()}


def run_reference(args):
    """Reference arm: the reference's own PyTorch attention (`_rel_attn`, staged under baseline/_ref/ by the
    build; its port in oracle/ where that is absent) on the box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = dict(WORKLOAD, B=1, H=4, Hkv=4)   # one batch element, 4 of its 16 heads per step
    for _ in range(min(args.warmup, 2)):
        cpu_port_time(dict(sample, H=1, Hkv=1))
    t0 = time.perf_counter()
    per, cores, kind = [], 1, "port"
    for _ in range(args.steps):
        t, cores, kind = cpu_port_time(sample)
        per.append(t)
    total = sum(per)
    f = flops(**sample)["f_alg"] * args.steps
    val = f / total / 1e12
    desc = "1 batch element x 4 heads of the workload per step (1/16 of it)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": NAME, "sample": desc},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }))


def make_inputs(torch, dev, w, seed, pinned=False):
    g = torch.Generator().manual_seed(seed)
    N = w["T"] * w["C"]
    B, H, Hkv, T, C, D = (w[k] for k in ("B", "H", "Hkv", "T", "C", "D"))
    shapes = dict(q=(B, H, N, D), u=(1, Hkv, 1, D), v=(1, Hkv, 1, D), z=(1, Hkv, 1, D), k=(B, Hkv, N, D),
                  rt=(1, Hkv, T, D), rc=(1, Hkv, C, D), val=(B, Hkv, N, D))
    host = {n: torch.randn(*s, generator=g).to(torch.bfloat16) for n, s in shapes.items()}
    if pinned:
        host = {n: x.pin_memory() for n, x in host.items()}
    return host, {n: x.to(dev) for n, x in host.items()}


def time_kernel(torch, attentions, t, w, steps, warmup, flush, gout=None):
    """Device time of `steps` calls; with `gout` (the gradient of the output) each call is forward + backward."""
    fwd = lambda: attentions.flashmvpa(t["q"], t["u"], t["v"], t["z"], t["k"], t["rt"], t["rc"], t["val"],
                                       causal=True, sm_scale=w["D"] ** -0.5, window_size=w["window"])
    if gout is None:
        call = fwd
    else:
        t = {n: x.detach().clone().requires_grad_(True) for n, x in t.items()}

        def call():
            for x in t.values():
                x.grad = None
            fwd().backward(gout)
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        flush.add_(1)          # writes 256 MiB: evicts the 126 MB L2 between timed launches
        a.record()
        call()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in ev]


def time_layer(torch, dev, flush, reps=10, warm=3):
    """The layer module (`layers/mvpa.py:341-409` in the reference) at one sample of BASELINE config 5:
    projections (cuBLAS) + the attention kernel on strided head views + `c_proj`.  Also times, on the same
    tensors, the head split / merge copies the reference layer makes (`layers/mvpa.py:383-390,398-399`)
    and this one does not."""
    from types import SimpleNamespace as NS
    import layers
    H, Hkv, D, T, C = 16, 8, 128, 128, 128
    E, N = H * D, T * C
    cfg = NS(max_position_embeddings=T, hidden_size=E, num_attention_heads=H, n_head_kv=Hkv, n_inner=5632,
             global_att=True, scale_attn_weights=True, scale_attn_by_inverse_layer_idx=False,
             reorder_and_upcast_attn=False, lora=False, attn_pdrop=0.0, resid_pdrop=0.0)
    torch.manual_seed(4)
    m = layers.MVPFormerGQAFlashAttention(cfg, layer_idx=0).eval().to(dev).to(torch.bfloat16)
    x = torch.randn(1, T, C, E, device=dev, dtype=torch.bfloat16)
    pos = torch.randn(1, T, E, device=dev, dtype=torch.bfloat16)
    chan = torch.randn(1, C, E, device=dev, dtype=torch.bfloat16)

    def timed(fn):
        ms = []
        for i in range(warm + reps):
            flush.add_(1)  # writes 256 MiB: evicts the L2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warm:
                ms.append(e0.elapsed_time(e1))
        return statistics.mean(ms)

    with torch.no_grad():
        layer_ms = timed(lambda: m(x, pos, chan))
        q = torch.randn(1, N, H, D, device=dev, dtype=torch.bfloat16)
        kv = torch.randn(1, N, 2 * Hkv, D, device=dev, dtype=torch.bfloat16)
        o = torch.randn(1, H, N, D, device=dev, dtype=torch.bfloat16)

        def copies():
            q.permute(0, 2, 1, 3).contiguous()
            kv[:, :, :Hkv].permute(0, 2, 1, 3).contiguous()
            kv[:, :, Hkv:].permute(0, 2, 1, 3).contiguous()
            o.permute(0, 2, 1, 3).contiguous()
        copies_ms = timed(copies)
    # training step of the layer: forward + backward (parameter and input gradients; gradients accumulate)
    xg, gout = x.clone().requires_grad_(True), torch.randn_like(x)
    train_ms = timed(lambda: m(xg, pos, chan)[0].backward(gout))
    return {"ms": layer_ms, "tokens_per_s": N / (layer_ms * 1e-3),
            "head_split_merge_copies_avoided_ms": copies_ms,
            "fwd_bwd_ms": train_ms, "fwd_bwd_tokens_per_s": N / (train_ms * 1e-3)}


MODELS = {
    # BASELINE config 4: MVPFormer-S classification (`configs/mvpformer_s_classification.yaml`), batch 8, 64 channels,
    # 128 segments of 2560 samples; n_positions raised from the YAML's 110 to 128 so that 128 segments have embeddings
    "cfg4": dict(arch=dict(n_embd=768, n_layer=12, n_head=12, n_head_kv=4, n_inner=1728), B=8, T=128, C=64, task="classify",
                 seed=3, tflop_per_sample=1.86, warm=3, steps=5),
    # BASELINE config 5: MVPFormer generative next-state forward (`configs/mvpformer_generative.yaml`), batch 32,
    # 128 channels x 128 segments (16384 tokens per sample)
    "cfg5": dict(arch=dict(n_embd=2048, n_layer=24, n_head=16, n_head_kv=8, n_inner=5632), B=32, T=128, C=128,
                 task="generative", seed=4, tflop_per_sample=53.2, warm=2, steps=2),
}


def time_model(torch, dist, dev, name, world, rank, flush):
    """Full-model forward (encoder -> MVPFormer stack -> head) on synthetic iEEG created on the device, the
    batch split across the ranks (batch elements are independent; no data-path collective).  Random-init
    weights of the named architecture, bf16.  Returns whole-job tokens/s (max time over ranks)."""
    import models
    from attentions import flash_mvpa_into
    from eeg_datasets import synthetic_ieeg
    spec = MODELS[name]
    a, T, C, n = spec["arch"], spec["T"], spec["C"], 2560
    warm, steps = spec["warm"], spec["steps"]   # the first calls carry one-off work (graph capture, lazy library set-up)
    B_total = spec["B"]
    B = B_total // world if B_total % world == 0 else 0
    if B == 0:
        return {"skipped": f"batch {B_total} does not split over {world} ranks"}
    E = a["n_embd"]
    torch.manual_seed(100 + spec["seed"])
    with torch.device(dev):
        cfg = models.MVPFormerConfig(n_positions=128, n_channels=128, **a)
        gen = spec["task"] == "generative"
        cls = models.HMVPFormer if gen else models.ClassificationHMVPFormer
        task = cls(cfg, models.WaveEncoder(n, E), models.MVPFormerHead(E, None if gen else 2), num_negatives=30)
    task = task.to(dev).to(torch.bfloat16).eval()
    task.mvpformer.enable_cuda_graph()                       # the block stack replays as one graph launch
    x = synthetic_ieeg(B, T, C, n, seed=1000 * spec["seed"] + rank, device=dev)   # fp32, in HBM
    neg = task._negative_indices((B, T, C), torch.Generator(device=dev).manual_seed(7)) if gen and B > 1 else None

    def step():
        if gen and B > 1:
            return task.next_state_logits(x, negatives=neg)
        if gen:                                            # one sample per rank: no other sample to draw negatives from
            out, _ = task._common_forward(x)
            return task.head(out)
        return task.classify(x)

    ms = []
    for i in range(warm + steps):
        flush.add_(1)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        y = step()
        e1.record()
        torch.cuda.synchronize()
        if i >= warm:
            ms.append(e0.elapsed_time(e1))
    finite = bool(torch.isfinite(y.float()).all())
    # share of the attention kernels: the same operator call on tensors of the layer's shapes, times the layer count
    H, Hkv = a["n_head"], a["n_head_kv"]
    D, N = E // H, T * C
    r = lambda *sh: torch.randn(*sh, device=dev, dtype=torch.bfloat16)
    q, k, v, o = r(B, N, H, D), r(B, N, Hkv, D), r(B, N, Hkv, D), r(B, N, H, D)
    small = (r(Hkv, D), r(Hkv, D), r(Hkv, D))
    rt, rc = r(Hkv, T, D), r(Hkv, C, D)
    att = []
    for i in range(4):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        flash_mvpa_into(o.permute(0, 2, 1, 3), q.permute(0, 2, 1, 3), *small, k.permute(0, 2, 1, 3), rt, rc,
                        v.permute(0, 2, 1, 3), D ** -0.5, 10)
        e1.record()
        torch.cuda.synchronize()
        if i >= 1:
            att.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.mean(ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms = float(t.item())
    del task, x
    torch.cuda.empty_cache()
    return {"ms": step_ms, "tokens_per_s": B_total * N / (step_ms * 1e-3), "global_batch": B_total, "per_gpu_batch": B,
            "tokens_per_sample": N, "share_of_attention": a["n_layer"] * statistics.mean(att) / statistics.mean(ms),
            "model_tflops_f_alg": spec["tflop_per_sample"] * B_total / (step_ms * 1e-3), "finite": finite,
            "input": "synthetic 1/f iEEG + 3-8 Hz bursts, fp32, generated on the device", "task": spec["task"],
            "cuda_graph": True}


def time_long_sample(torch, dist, dev, world, rank, flush, one_gpu_ms):
    """One 16k-token sample (D 128, 16 heads / 8 kv heads) with its time axis spread over the ranks: every rank
    holds the q / k|v rows of its two zig-zag chunks, K and V are gathered over NVLink on a communication
    stream in two halves - by NCCL collectives, and by the library's own peer-load kernel ordered by flags
    between the GPUs - and the rank's two query ranges run against the gathered K/V; the early range starts
    when the early half has landed.  Strong scaling against the single-GPU forward of the sample."""
    import attentions
    import mvpa_shard as ms
    w = WORKLOADS["16k"][0]
    H, Hkv, T, C, D = (w[k] for k in ("H", "Hkv", "T", "C", "D"))
    plan = ms.zigzag_chunks(T, C, world)
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    r = lambda *sh: torch.randn(*sh, device=dev, dtype=torch.bfloat16, generator=g)
    q_loc = [r(1, n * C, H, D) for _, n in plan[rank]]
    kv_loc = [r(1, n * C, 2 * Hkv, D) for _, n in plan[rank]]
    g2 = torch.Generator(device=dev).manual_seed(49)          # replicated small tensors: same on every rank
    r2 = lambda *sh: torch.randn(*sh, device=dev, dtype=torch.bfloat16, generator=g2)
    u, vt, z, rt, rc = r2(1, Hkv, 1, D), r2(1, Hkv, 1, D), r2(1, Hkv, 1, D), r2(1, Hkv, T, D), r2(1, Hkv, C, D)
    kw = dict(dim=D, dtype=torch.bfloat16, device=dev, batch=1)

    def timed(fn, reps=6, warm=2):
        out = []
        for i in range(warm + reps):
            dist.barrier()
            torch.cuda.synchronize()
            # The L2 flush runs right before the timed region, three times: while the GPU is busy with it the
            # host enqueues the step, so the events see the device time of the step and not the time Python
            # takes to launch a dozen small operations onto an idle GPU (a model's host thread runs ahead of
            # the GPU in the same way; the single-GPU time this is compared with is taken behind a flush too).
            for _ in range(3):
                flush.add_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warm:
                out.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.mean(out)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.no_grad():
        total = timed(lambda: ms.time_sharded_attention(attentions.flashmvpa, q_loc, u, vt, z, kv_loc, rt, rc, None, T, C,
                                                        D ** -0.5, 10))
        gather = timed(lambda: ms.gather_kv(kv_loc, plan, T, C, heads=2 * Hkv, **kw))
        # the same with this library's peer-load gather kernel (CUDA IPC mappings of the ranks' send buffers)
        # instead of the NCCL collectives
        try:
            p2p = {"ms": timed(lambda: ms.time_sharded_attention(attentions.flashmvpa, q_loc, u, vt, z, kv_loc, rt, rc, None,
                                                                  T, C, D ** -0.5, 10, transport="p2p")),
                   "gather_ms": timed(lambda: ms.gather_kv(kv_loc, plan, T, C, heads=2 * Hkv, transport="p2p", **kw))}
            p2p["speedup_vs_1gpu"] = one_gpu_ms / p2p["ms"]
        except Exception as e:      # e.g. ranks that cannot map one another's memory
            p2p = {"unavailable": repr(e)[:200]}
        full = ms.gather_kv(kv_loc, plan, T, C, heads=2 * Hkv, **kw)
        kf, vf = full[:, :, :Hkv].permute(0, 2, 1, 3), full[:, :, Hkv:].permute(0, 2, 1, 3)

        def attn_only():
            for (t0, n), ql in zip(plan[rank], q_loc):
                attentions.flashmvpa(ql.permute(0, 2, 1, 3), u, vt, z, kf, rt, rc, vf, causal=True, sm_scale=D ** -0.5,
                                     window_size=10, q_time_range=(t0, n))
        attn = timed(attn_only)
    nccl = {"ms": total, "gather_ms": gather, "speedup_vs_1gpu": one_gpu_ms / total}
    best = p2p if "ms" in p2p else nccl          # the library's own transport where the ranks can map one another's memory
    return {"ms": best["ms"], "tokens_per_s": T * C / (best["ms"] * 1e-3), "gather_ms": best["gather_ms"],
            "attention_only_ms": attn, "exposed_gather_ms": max(0.0, best["ms"] - attn),
            "speedup_vs_1gpu": one_gpu_ms / best["ms"], "one_gpu_ms": one_gpu_ms,
            "gathered_bytes_per_rank": 2 * Hkv * D * 2 * T * C * (world - 1) // world,
            "transport": "peer loads over NVLink (mvpa_peer_gather + flags)" if best is p2p else "nccl",
            "nccl_transport": nccl, "peer_load_transport": p2p,
            "timing": "device time: the step is enqueued behind the L2 flush, like the single-GPU forward it is compared with",
            "limiter": "the K/V gather before a rank's late query range can start, and the query tile of the last time "
                       "steps, which walks all 128 key tiles in one CTA"}


def time_long_sample_model(torch, dist, dev, world, rank, flush):
    """The block stack of BASELINE config 5 (24 layers, E 2048, 16 heads / 8 kv heads) on ONE 16k-token sample:
    the fused forward on one GPU against `forward_time_sharded` with the sample's time axis spread over the
    ranks (zig-zag chunks; per layer only K and V travel, through the library's peer-load kernels, while the
    MLP gate runs).  Random-init weights, encoder outputs drawn on the device.  Strong scaling of one sample."""
    import models
    import mvpa_shard as ms
    spec = MODELS["cfg5"]
    a, T, C = spec["arch"], spec["T"], spec["C"]
    E = a["n_embd"]
    torch.manual_seed(777)                                    # the same weights on every rank
    with torch.device(dev):
        cfg = models.MVPFormerConfig(n_positions=128, n_channels=128, **a)
        model = models.MVPFormerModel(cfg)
    model = model.to(dev).to(torch.bfloat16).eval()
    g = torch.Generator(device=dev).manual_seed(778)
    emb = (torch.randn(1, T, C, E, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    plan = ms.zigzag_chunks(T, C, world)
    mine = torch.cat([emb.view(T * C, E)[t0 * C:(t0 + n) * C] for t0, n in plan[rank]])

    def timed(fn, reps=3, warm=2):
        out = []
        for i in range(warm + reps):
            dist.barrier()
            torch.cuda.synchronize()
            flush.add_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            y = fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warm:
                out.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.mean(out)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), y

    with torch.no_grad():
        one, ref = timed(lambda: model(inputs_embeds=emb).last_hidden_state)
        res = {}
        ref = ref.view(T * C, E)
        want = torch.cat([ref[t0 * C:(t0 + n) * C] for t0, n in plan[rank]]).float()
        for transport in ("p2p_graph", "p2p", "nccl"):
            try:
                kw = dict(transport="p2p", graph=True) if transport == "p2p_graph" else dict(transport=transport)
                ms_t, got = timed(lambda: model.forward_time_sharded(mine, T, C, **kw))
                err = torch.tensor([float((got.float() - want).abs().max())], dtype=torch.float64, device=dev)
                dist.all_reduce(err, op=dist.ReduceOp.MAX)
                res[transport] = {"ms": ms_t, "speedup_vs_1gpu": one / ms_t, "tokens_per_s": T * C / (ms_t * 1e-3),
                                  "max_abs_diff_vs_1gpu": float(err.item())}
            except Exception as e:
                res[transport] = {"unavailable": repr(e)[:200]}
    best = next(res[k] for k in ("p2p_graph", "p2p", "nccl") if "ms" in res[k] or k == "nccl")
    return {"one_gpu_ms": one, "ms": best.get("ms"), "speedup_vs_1gpu": best.get("speedup_vs_1gpu"),
            "tokens_per_s": best.get("tokens_per_s"), "layers": a["n_layer"], "tokens": T * C,
            "peer_load_transport_cuda_graph": res["p2p_graph"], "peer_load_transport": res["p2p"],
            "nccl_transport": res["nccl"],
            "hidden_state_scale": float(want.abs().max())}


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier pool measurement)"


def run_blocks(args):
    """`--workload blocks`: the HBM-bound kernels around the attention (RMSNorm with and without the residual
    add, SwiGLU gate, wavelet encoder front end, readouts) at the shapes one rank of BASELINE config 5 on 8 GPUs
    sees (4 samples x 16384 tokens, E 2048, I 5632, segments of 2560 samples).  Per kernel: device time by CUDA
    events, algorithmic bytes (every input read once, every output written once), GB/s against the measured copy
    bandwidth.  One JSON line."""
    import torch
    import mvpa_native
    import mvpa_ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = mvpa_native.lib()
    M, E, I, n, K = args.block_tokens, 2048, 5632, 2560, 30
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    r = lambda *sh, dt=bf: torch.randn(*sh, device=dev, dtype=torch.float32, generator=g).to(dt)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    x, a, w = r(M, E), r(M, E), r(E)
    big = r(M, 2 * I)
    act = torch.empty(M, I, device=dev, dtype=bf)
    sig = r(M, n, dt=torch.float32)
    _, total = mvpa_ops.wave_sizes(n)
    lnw = r(total)
    B, T, C = max(2, M // 16384), 128, 128
    pred, enc = r(B, T, C, E), r(B, T, C, E)
    neg = torch.randint(0, B * T * C, (B, T, C, K), device=dev, dtype=torch.int32, generator=g)
    h = x.clone()
    cases = {
        "rmsnorm_kernel (ln_1 / ln_f)": (lambda: mvpa_ops.rmsnorm(x, w, 1e-5), 2 * M * E * 2),
        "rmsnorm_kernel (+ residual add)": (lambda: mvpa_ops.rmsnorm(h, w, 1e-5, add=a, sum_out=h), 4 * M * E * 2),
        "silu_mul_kernel": (lambda: mvpa_ops.silu_mul(big[:, :I], big[:, I:], act), 3 * M * I * 2),
        "wave_encode_kernel": (lambda: mvpa_ops.wave_encode(sig, lnw, 1e-5, pad_to=2624), M * (n * 4 + 2624 * 2)),
        "channel_mean_kernel": (lambda: mvpa_ops.channel_mean(pred), B * C * E * 2 + B * E * 2),
        "contrastive_kernel (K = 30; negatives mostly from the L2)": (
            lambda: mvpa_ops.contrastive_logits(pred, enc, neg, 0.1), B * (T - 1) * C * ((K + 2) * E * 2 + (K + 1) * 4)),
    }
    peak, src = hbm_peak()
    n0 = lib.mvpa_launch_count()
    out = {}
    for name, (fn, nbytes) in cases.items():
        ms = []
        for i in range(3 + args.steps):
            flush.add_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                ms.append(e0.elapsed_time(e1))
        m = statistics.mean(ms)
        out[name] = {"ms": m, "algorithmic_bytes": nbytes, "gb_per_s": nbytes / m / 1e6, "frac_of_hbm_peak": nbytes / m / 1e6 / peak}
    print(json.dumps({"workload": f"blocks: kernels around the attention at config 5's per-rank shapes (M {M} tokens, E 2048, I 5632)",
                      "bound": "hbm", "peak_gb_per_s": peak, "peak_source": src, "steps": args.steps,
                      "gpu_launches": int(lib.mvpa_launch_count() - n0), "kernels": out}))


def run_triton(args):
    """The reference's own Triton operator (`attentions/attn.py:1317-1366`, unmodified, loaded from
    baseline/_ref/attentions/) on this GPU: first a small shape checked against this library, then the
    benchmark workload.  Any failure to compile or launch is reported as text."""
    import importlib.util
    import traceback
    out = {"impl": "triton", "workload": NAME}
    try:
        import torch
        import attentions
        path = os.path.join(ROOT, "baseline", "_ref", "attentions", "attn.py")
        if not os.path.exists(path):
            out["unavailable"] = "baseline/_ref/attentions/attn.py is not staged"
            print(json.dumps(out))
            return
        import triton
        out["triton_version"] = triton.__version__
        spec = importlib.util.spec_from_file_location("reference_attentions_attn", path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        small = dict(B=1, H=2, Hkv=2, T=16, C=16, D=64, window=10)
        for stage, w in (("small", small), ("workload", WORKLOAD)):
            _, t = make_inputs(torch, dev, w, seed=1)
            call = lambda f: f(t["q"], t["u"], t["v"], t["z"], t["k"], t["rt"], t["rc"], t["val"], causal=True,
                               sm_scale=w["D"] ** -0.5, window_size=w["window"])
            with torch.no_grad():
                o_ref = call(ref.flash_mvpa)
                torch.cuda.synchronize()
                o_own = call(attentions.flashmvpa)
                out[stage + "_max_abs_diff_vs_this_library"] = float((o_ref.float() - o_own.float()).abs().max())
        flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device=dev)
        ms = []
        with torch.no_grad():
            for i in range(3 + args.steps):
                flush.add_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                call(ref.flash_mvpa)
                e1.record()
                torch.cuda.synchronize()
                if i >= 3:
                    ms.append(e0.elapsed_time(e1))
        f = flops(**WORKLOAD)
        m = statistics.mean(ms)
        out.update(ms=m, tflops_f_alg=f["f_alg"] / m / 1e9, tflops_f_dense=f["f_dense"] / m / 1e9, steps=len(ms),
                   includes="_rel_bias (two cuBLAS products into HBM) + _fwd_kernel, as the reference operator runs them")
    except BaseException as e:  # the error text is the data point
        out["error"] = f"{type(e).__name__}: {e}"[:1500]
        out["traceback_tail"] = traceback.format_exc()[-1500:]
    print(json.dumps(out))


def triton_point(args, device_index):
    """Runs `--impl triton` in a child process (a compiler crash or a long compile must not take the benchmark
    with it) and returns its JSON."""
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR",
                                                             "MASTER_PORT", "OMP_NUM_THREADS")}
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    ids = [x for x in vis.split(",") if x.strip()] if vis else None
    env["CUDA_VISIBLE_DEVICES"] = ids[device_index] if ids and device_index < len(ids) else str(device_index)
    try:
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "triton", "--workload", args.workload,
                              "--steps", "10"], capture_output=True, text=True, timeout=600, env=env)
        for line in reversed(res.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
        return {"impl": "triton", "error": "no JSON line", "stderr_tail": res.stderr[-1200:], "returncode": res.returncode}
    except subprocess.TimeoutExpired:
        return {"impl": "triton", "error": "child process exceeded 600 s (compile or run); not retried"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "triton"],
                    help="reference: the CPU arm; triton: the reference's Triton operator on this GPU (an extra point)")
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + ["blocks"],
                    help="cfg2 is the benchmark; the others exist for profiling and extra points "
                         "(blocks: the HBM-bound kernels around the attention)")
    ap.add_argument("--pass", dest="passes", default="fwd", choices=["fwd", "fwd_bwd"],
                    help="fwd is the benchmark; fwd_bwd times forward + backward (training step of the operator)")
    ap.add_argument("--block-tokens", type=int, default=65536, help="rows of the `blocks` workload (profiling uses fewer)")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra reported points")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "blocks":
        return run_blocks(args)
    global WORKLOAD, NAME
    WORKLOAD, NAME = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "triton":
        return run_triton(args)

    import torch
    import torch.distributed as dist
    import attentions
    import mvpa_native

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = mvpa_native.lib()
    w = WORKLOAD
    host, t = make_inputs(torch, dev, w, seed=1 + rank, pinned=True)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    f = flops(**w)
    train = args.passes == "fwd_bwd"
    gout = torch.randn(t["q"].shape, device=dev, dtype=torch.bfloat16) if train else None
    if train:  # flops of the step: forward + backward
        fb = flops_bwd(**w)
        f = {"f_alg": f["f_alg"] + fb, "f_dense": f["f_dense"] + fb}

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ----
    sync_all()
    n0 = lib.mvpa_launch_count()
    clk = ClockSampler(local)
    clk.__enter__()
    sync_all()
    ms = time_kernel(torch, attentions, t, w, args.steps, args.warmup, flush, gout)
    sync_all()
    per_call = (lib.mvpa_launch_count() - n0) // (args.steps + args.warmup)  # kernels of the library per call
    launches = per_call * args.steps
    total_ms = torch.tensor([sum(ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    value = world * f["f_alg"] * args.steps / (total_ms * 1e-3) / 1e12

    # ---- end to end: pinned host inputs -> device -> flashmvpa -> host ----
    big = ("q", "k", "val")
    o_host = torch.empty(host["q"].shape, dtype=torch.bfloat16).pin_memory()
    gout_host = gout.cpu().pin_memory() if train else None
    h2d = sum(host[n].numel() * 2 for n in host) + (gout_host.numel() * 2 if train else 0)
    d2h = o_host.numel() * 2

    # Three streams and two sets of device buffers: the host->device copy of step i+1, the kernels of
    # step i and the device->host copy of step i-1 overlap, as in a serving loop fed from pinned memory.
    # Every step's copies and kernels are inside the timed region.
    s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    NBUF = 2
    dbuf = [{n: torch.empty_like(t[n]) for n in host} for _ in range(NBUF)]
    gbuf = [torch.empty_like(gout) for _ in range(NBUF)] if train else None
    obuf = [torch.empty_like(t["q"]) for _ in range(NBUF)]
    ev_in = [torch.cuda.Event() for _ in range(NBUF)]      # inputs of the buffer have landed
    ev_run = [torch.cuda.Event() for _ in range(NBUF)]     # kernels reading / writing the buffer are done
    ev_out = [torch.cuda.Event() for _ in range(NBUF)]     # the result has left the buffer

    def e2e_step(i):
        j = i % NBUF
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_run[j])                      # the kernels of step i - NBUF no longer read these inputs
            for n in host:
                dbuf[j][n].copy_(host[n], non_blocking=True)
            if train:
                gbuf[j].copy_(gout_host, non_blocking=True)
            ev_in[j].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[j])
            s_run.wait_event(ev_out[j])                     # the result of step i - NBUF has been copied out
            d = dbuf[j]
            if train:
                d = {n: x.detach().requires_grad_(True) for n, x in d.items()}
            o = attentions.flashmvpa(d["q"], d["u"], d["v"], d["z"], d["k"], d["rt"], d["rc"], d["val"],
                                     causal=True, sm_scale=w["D"] ** -0.5, window_size=w["window"])
            if train:  # the step's result read back is dq
                o.backward(gbuf[j])
                obuf[j].copy_(d["q"].grad)
            else:
                obuf[j].copy_(o)
            ev_run[j].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[j])
            o_host.copy_(obuf[j], non_blocking=True)
            ev_out[j].record(s_out)

    for i in range(args.warmup):
        e2e_step(i)
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()                                               # default stream: the side streams start after it
    for st in (s_in, s_run, s_out):
        st.wait_stream(torch.cuda.current_stream())
    for i in range(args.steps):
        e2e_step(i)
    for st in (s_in, s_run, s_out):
        torch.cuda.current_stream().wait_stream(st)
    b.record()
    sync_all()
    clk.__exit__()
    e2e_ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_val = world * f["f_alg"] * args.steps / (float(e2e_ms.item()) * 1e-3) / 1e12

    if rank == 0:
        peak, peak_src = peaks(sustained=args.workload == "cfg5")
        kernel_ms = statistics.mean(ms)
        achieved = f["f_alg"] / (kernel_ms * 1e-3) / 1e12
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": NAME + (" (forward + backward)" if train else ""), "per_gpu_batch": w["B"], "global_batch": w["B"] * world,
                       "l2": "256 MiB buffer rewritten between timed launches", "parallelism": f"batch x{world}"},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": None if train else NCU_DRAM_BYTES.get(args.workload), "peak_source": peak_src,
                         "kernel": ("whole step (tc_fwd_kernel, tc_bwd_q_kernel, tc_bwd_kv_kernel, simt_drel_kernel)"
                                    if train else "tc_fwd_kernel<%d,%d>" %
                                    (w["D"], 32 if w["C"] <= 32 else 64 if w["C"] <= 64 else 128)),
                         "flops_per_launch": f["f_alg"],
                         "achieved_dense_convention": f["f_dense"] / (kernel_ms * 1e-3) / 1e12},
        }
        out["roofline"]["traffic_source"] = "ncu capture summarised under profiles/ (not measured in this run)"
    extra, ms_16k = {}, None
    if not args.no_extra:  # points every rank takes part in
        for name in ("cfg4", "cfg5"):
            res = time_model(torch, dist, dev, name, world, rank, flush)
            extra["model_" + name] = res
        _, tt = make_inputs(torch, dev, WORKLOADS["16k"][0], seed=7)
        ms_16k = statistics.mean(time_kernel(torch, attentions, tt, WORKLOADS["16k"][0], 10, 3, flush))
        del tt
        if world > 1:
            extra["long_sample_16k"] = time_long_sample(torch, dist, dev, world, rank, flush, ms_16k)
            extra["model_long_sample_16k"] = time_long_sample_model(torch, dist, dev, world, rank, flush)
    if rank == 0:
        if not args.no_extra:
            ff = flops(**WORKLOADS["16k"][0])
            out["roofline"]["north_star_16k"] = {
                "workload": WORKLOADS["16k"][1], "ms": ms_16k, "achieved": ff["f_alg"] / ms_16k / 1e9,
                "frac": ff["f_alg"] / ms_16k / 1e9 / peak, "target_frac": 0.60,
                "achieved_dense_convention": ff["f_dense"] / ms_16k / 1e9}
            for name, ww in (("16k_tokens_D128_H16_Hkv8_B1", WORKLOADS["16k"][0]),
                             ("cfg3_fwd_B8_T128_C32_D64", WORKLOADS["cfg3"][0])):
                _, tt = make_inputs(torch, dev, ww, seed=7)
                m2 = ms_16k if ww is WORKLOADS["16k"][0] else statistics.mean(time_kernel(torch, attentions, tt, ww, 10, 3, flush))
                ff = flops(**ww)
                extra[name] = {"ms": m2, "tflops_f_alg": ff["f_alg"] / m2 / 1e9, "tflops_f_dense": ff["f_dense"] / m2 / 1e9,
                               "frac_of_peak_f_alg": ff["f_alg"] / m2 / 1e9 / peak}
                del tt
            # training path: forward + backward through autograd, dO ~ N(0,1)
            for name, ww in (("cfg3_fwd_bwd_B8_T128_C32_D64", WORKLOADS["cfg3"][0]),
                             ("16k_tokens_fwd_bwd_D128_H16_Hkv8_B1", WORKLOADS["16k"][0])):
                _, tt = make_inputs(torch, dev, ww, seed=2)
                g2 = torch.randn(tt["q"].shape, device=dev, dtype=torch.bfloat16)
                m3 = statistics.mean(time_kernel(torch, attentions, tt, ww, 10, 3, flush, g2))
                f3 = flops(**ww)["f_alg"] + flops_bwd(**ww)
                extra[name] = {"ms": m3, "tflops_f_alg": f3 / m3 / 1e9, "frac_of_peak_f_alg": f3 / m3 / 1e9 / peak}
                del tt, g2
            extra["layer_fwd_16k_tokens_E2048_H16_Hkv8"] = time_layer(torch, dev, flush)
            if world == 1:  # the reference's Triton operator on this GPU, in a child process
                extra["triton_reference"] = triton_point(args, local)
                if not args.no_cpu:
                    extra["cpu_config1"] = cpu_config1()
            out["extra"] = extra
        if not args.no_cpu and world == 1:  # the CPU leg belongs to the single-GPU run
            sample = dict(w, B=1)
            cpu_port_time(dict(sample, H=1, Hkv=1))  # warm-up: thread pool, allocator
            sec, cores, kind = cpu_port_time(sample, reps=10)  # about 10 s of CPU work
            out["cpu_baseline"] = {"value": flops(**sample)["f_alg"] / sec / 1e12, "unit": UNIT, "cores": cores,
                                   "kind": kind, "sample": "1 of the 4 batch elements (16 heads, 4096 tokens), fp32, median of 10 passes",
                                   "seconds": sec}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
