#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the half-depth Flint configuration (24 layers, hidden 2048,
32 query / 4 KV heads of 128, 256 experts of width 512, top-8, vocabulary 151,936) with random
weights, a batch of 8 requests that each hold 32,768 cached tokens, bfloat16.  One JSON line:
`value` is decoded tokens a second timed on the device (CUDA events around K decode steps of
ModelRunner.step plus the device argmax); `e2e` is the same through Engine.step() with host token
ids in (pinned host memory -> device) and sampled ids out (device -> host) every step; `prefill`
is one 2,048-token prompt in one step; `points` are decode at batch 1 and 64; `roofline` is the
decode step's bytes (every weight it uses once, and the cache of the live requests) over its time
over the peak copy bandwidth.  Peaks come from MEASURED_PEAKS.json beside this file when the
measuring harness wrote it, else from the fallback figures below.

The caches are filled with random values instead of by a prefill (the weights are random too), so
every request stands at the context length at once; what the decode step reads and computes is the
same.  Inputs are larger than L2: one decode step streams gigabytes of weights and cache.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

CONFIG2 = {
    "architectures": ["FlintForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 24, "num_attention_heads": 32,
    "num_key_value_heads": 4, "head_dim": 128, "vocab_size": 151936, "n_routed_experts": 256, "num_experts_per_tok": 8,
    "moe_intermediate_size": 512, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "kv_page_size": 16,
}


# the further shapes this file can run: the full-depth model (about 80 GB of weights) at 8,192 cached tokens
SHAPES = {2: {"layers": 24, "context": 32768, "label": "Recursive Flint MoE, half-depth shape"},
          3: {"layers": 48, "context": 8192, "label": "Recursive Flint MoE, 40B-A2.5B shape"}}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in d.items() if k in out and isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons of GPU 0 while a timed region runs: read through NVML every
    5 ms when its Python binding is there (a timed region of a few dozen milliseconds still gets
    several samples), else from `nvidia-smi -lms 200`.  Reading only; nothing is set."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.lines, self.proc, self.nvml, self.samples, self.stop_flag = [], None, None, [], False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
                                                            if os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].isdigit() else 0)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(reasons_fn(self.handle))
                self.samples.append((mhz, {n for n, b in bits.items() if mask & b}))
            except Exception:
                pass
            time.sleep(0.005)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1)
            sm = sorted(m for m, _ in self.samples)
            reasons = set().union(*[r for _, r in self.samples]) if self.samples else set()
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(self.NAMES, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def expected_experts(E, k, B):
    return E * (1.0 - (1.0 - k / E) ** B)


def decode_bytes(cfg, layers, B, ctx, experts_read=None):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests.
    experts_read: distinct experts per layer that the router really chose (measured); else the expectation."""
    D, Hq, Hkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, I, V = cfg["n_routed_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["vocab_size"]
    attn = ((Hq + 2 * Hkv) * hd * D + D * Hq * hd) * 2
    router = E * D * 2
    experts = (experts_read if experts_read is not None else expected_experts(E, k, B)) * 3 * I * D * 2
    weights = layers * (attn + router + experts) + V * D * 2
    kv = B * ctx * layers * 2 * Hkv * hd * 2
    return weights + kv, weights, kv


def prefill_bytes(cfg, layers, T):
    """Bytes a prefill step of T tokens has to read at least: every weight once (with T * k pairs far above the number of
    experts, all of them), the logits' row of the head aside."""
    D, Hq, Hkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, I, V = cfg["n_routed_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["vocab_size"]
    per_layer = ((Hq + 2 * Hkv) * hd * D + D * Hq * hd + E * D + expected_experts(E, k, T) * 3 * I * D) * 2
    return layers * per_layer + V * D * 2


def prefill_flops(cfg, layers, T):
    D, Hq, Hkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, I, V = cfg["n_routed_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["vocab_size"]
    per_token = (Hq + 2 * Hkv) * hd * D + D * Hq * hd + E * D + k * 3 * I * D
    matmul = 2.0 * T * layers * per_token + 2.0 * V * D
    attention = layers * 4.0 * Hq * hd * T * (T / 2.0)
    return matmul + attention


def kernel_attention_prefill(args):
    """The prompt-portion attention kernel alone: T query tokens of one request whose last token stands
    at position `context - 1`, over a cache of `context` keys (so T = context is a whole prompt from
    position 0); FLOPs counted under the causal mask; CUDA events, warm-up, cache larger than L2 from
    32,768 keys on."""
    import torch
    from quench6k_b200 import ops
    from quench6k_b200.engine.batch import StepContext
    c = CONFIG2
    Hq, Hkv, hd, ps = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], args.page_size or c["kv_page_size"]
    n, T, dev = args.context, min(args.prefill_tokens, args.context), "cuda:0"
    pages = (n + ps - 1) // ps
    kp = torch.randn(Hkv, pages, ps, hd, device=dev).to(torch.bfloat16)
    vp = torch.randn(Hkv, pages, ps, hd, device=dev).to(torch.bfloat16)
    q = torch.randn(T, Hq, hd, device=dev).to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ctx = StepContext(T=T, R=1, token_ids=i32([0] * T), positions=i32(list(range(n - T, n))), req_of_token=i32([0] * T), q_start=i32([0, T]),
                      pos_start=i32([n - T]), slot_ids=i32([0]), block_tables=[i32([list(range(pages))])], logit_rows=i32([]), n_logit_rows=0,
                      q_lens=[T], pos_starts=[n - T], slots=[0], max_context=n, max_q_len=T)
    tok0, ntok, n_tiles = ctx.query_tile_pairs(ops.attention_tc_tile_tokens(Hq // Hkv), False)
    run = lambda: ops.attention_tc(q, kp, vp, ctx.block_tables[0], ctx.req_of_token, ctx.positions, tok0, ntok, None, None)
    for _ in range(max(3, args.warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * Hq * hd * T * (n - T + (T + 1) / 2.0)
    pk = peaks()
    print(json.dumps({"kernel": "attention_tc (prompt portions)", "tokens": T, "context": n, "us": round(ms * 1e3, 1),
                      "tflops": round(flops / ms / 1e9, 1), "frac_of_bf16_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3),
                      "peaks": pk["source"], "ctas": n_tiles * Hkv, "steps": args.steps}))
    return 0


def kernel_gated_delta(args):
    """The gated delta rule recurrence alone (with the kernel that prepares its per-token inputs): one request's portion of
    --prefill-tokens tokens, 16 heads of 128 x 128 on 4 key heads, or --batch requests of one token each (a decode step);
    CUDA events after warm-up.  Counted: 3 passes of 2 dk dv FLOPs per token and head (two sums over the state, one write)."""
    import torch
    from quench6k_b200 import ops
    H, G, dk, dv, dev = 16, 4, 128, 128, "cuda:0"
    decode = bool(args.batch)
    R, n = (args.batch, 1) if decode else (1, args.prefill_tokens)
    T = R * n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    u = torch.randn(T, 2 * G * dk + H * dv, device=dev)
    p = torch.randn(T, 2 * H, device=dev)
    A_log, dt_bias = torch.randn(H, device=dev) - 3.0, torch.randn(H, device=dev)
    state = torch.zeros(R, H, dv, dk, device=dev)
    q_start, slots = i32([i * n for i in range(R + 1)]), i32(list(range(R)))
    run = lambda: ops.gated_delta(u.clone() if not decode else u, p, 0, H, A_log, dt_bias, state, q_start, slots, R, H, G, dk, dv, prepare=n > 16)
    for _ in range(max(3, args.warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 6.0 * dk * dv * H * T
    state_bytes = 2.0 * 4 * H * dk * dv * R
    print(json.dumps({"kernel": "gated_delta", "requests": R, "tokens_each": n, "us": round(ms * 1e3, 1), "ns_per_token": round(ms * 1e6 / n, 1),
                      "gflops": round(flops / ms / 1e6, 1), "state_gbs": round(state_bytes / ms / 1e6, 1), "steps": args.steps,
                      "note": "prompt portions include a device copy of the inputs (the kernel normalises q and k in place)"}))
    return 0


def kernel_retention(args):
    """The retention recurrence alone: one request's portion of --prefill-tokens tokens, 16 heads of 128 x 128, or --batch
    requests of one token each (a decode step); CUDA events after warm-up.  Counted: 2 passes of 2 dk dv FLOPs per token
    and head (the state's update and its product with q); bytes: the state read and written, q, k, v read and o written."""
    import torch
    from quench6k_b200 import ops
    H, dk, dv, dev = 16, 128, 128, "cuda:0"
    decode = bool(args.batch)
    R, n = (args.batch, 1) if decode else (1, args.prefill_tokens)
    T = R * n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    p = torch.randn(T, 2 * H * dk + 2 * H * dv, device=dev) * 0.1
    decay = 1.0 - 2.0 ** (-5.0 - 5.0 * torch.arange(H, device=dev, dtype=torch.float32) / H)
    state = torch.zeros(R, H, dk, dv, device=dev)
    q_start, slots = i32([i * n for i in range(R + 1)]), i32(list(range(R)))
    run = lambda: ops.retention(p, 0, H * dk, 2 * H * dk, decay, state, q_start, slots, R, H, dk, dv)
    for _ in range(max(3, args.warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * dk * dv * H * T
    nbytes = 2.0 * 4 * H * dk * dv * R + 4.0 * T * H * (2 * dk + 2 * dv)
    print(json.dumps({"kernel": "retention", "requests": R, "tokens_each": n, "us": round(ms * 1e3, 1), "ns_per_token": round(ms * 1e6 / n, 1),
                      "gflops": round(flops / ms / 1e6, 1), "gbs": round(nbytes / ms / 1e6, 1), "steps": args.steps}))
    return 0


def profile_ops(args, runner, cfg_d, layers, ctx, stand_at_context, rand_ids):
    """Where the time of an eager decode step (batch --batch at the context) and of a prefill step goes, launcher by
    launcher: CUDA events around every launch (quench6k_b200.ops.profile_begin/profile_end), no profiler involved.  Eager
    launches leave gaps that a replayed graph does not have, so the sum is the step's kernel time, not its duration."""
    import torch
    from quench6k_b200 import ops
    from quench6k_b200.engine import StepEntry
    runner.cuda_graphs = False
    B, T = args.batch, args.prefill_tokens
    rids = [f"q{i}" for i in range(B)]
    stand_at_context(rids)
    toks = [rand_ids(args.steps + args.warmup) for _ in rids]
    step = lambda i: runner.step([StepEntry(r, [toks[j][i]], [0]) for j, r in enumerate(rids)])
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    ops.profile_begin()
    for i in range(args.warmup, args.warmup + args.steps):
        step(i)
    decode = ops.profile_end()
    for r in rids:
        runner.end_request(r)
    prefill = {}
    for it in range(2):
        runner.add_request("p")
        ids = rand_ids(T)
        if it:
            ops.profile_begin()
        runner.step([StepEntry("p", ids, [T - 1])])
        if it:
            prefill = ops.profile_end()
        runner.end_request("p")
    table = lambda rec, n: [{"op": tag, "launcher": fn, "calls_per_step": calls / n, "us_per_step": round(ms * 1e3 / n, 1)}
                            for (tag, fn), (calls, ms) in rec.items()]
    print(json.dumps({"profile": "CUDA events around every launch of eager steps", "layers": layers, "batch": B, "context": ctx,
                      "decode_step": table(decode, args.steps), "decode_us": round(sum(ms for _, ms in decode.values()) * 1e3 / args.steps, 1),
                      "prefill_tokens": T, "prefill_step": table(prefill, 1), "prefill_us": round(sum(ms for _, ms in prefill.values()) * 1e3, 1)}))
    return 0


# ---------------------------------------------------------------------------------------------- another design beside Flint
def pedotar_config(size):
    """Pedotar at layer sizes that resemble a real model's: per pass a selective scan, attention over a cached latent, chunked
    attention with mixed heads and another scan, the attention layers with a dense feed-forward; the span runs twice."""
    D, ff, inner, rank, heads, kv, chunk = {"s": (1024, 4096, 2048, 256, 8, 2, 512), "m": (2048, 8192, 4096, 512, 16, 4, 1024)}[size]
    scan = {"type": "mamba1", "mixer": {"inner": inner, "state": 16, "conv": 4, "dt_rank": D // 16}, "mlp": None}
    latent = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
              "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": rank, "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}}
    chunked = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
               "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": chunk}}}
    return {"architecture": "Pedotar", "vocab": 32768, "width": D, "norm": {"eps": 1e-6}, "kv_page_size": 16,
            "layers": [scan, latent, chunked, dict(scan)], "loop": {"start": 0, "stop": 4, "times": 2}}


def flint_dense_config(size):
    """The closest existing model at equal size: Flint with dense feed-forwards only, the same width, heads, feed-forward
    width, vocabulary and number of executed layers."""
    D, ff, _, _, heads, kv, _ = {"s": (1024, 4096, 0, 0, 8, 2, 0), "m": (2048, 8192, 0, 0, 16, 4, 0)}[size]
    return {"architectures": ["FlintForCausalLM"], "hidden_size": D, "num_hidden_layers": 8, "num_attention_heads": heads,
            "num_key_value_heads": kv, "head_dim": 128, "vocab_size": 32768, "n_routed_experts": 8, "num_experts_per_tok": 2,
            "moe_intermediate_size": 64, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "first_k_dense_replace": 8,
            "intermediate_size": ff, "kv_page_size": 16}


def kipedra_config(size):
    """Kipedra at layer sizes that resemble a real model's: a gated delta rule layer with a dense feed-forward, two layers of
    windowed attention with routed experts and a delta layer with routed experts; the four run twice."""
    D, ff, heads, kv, E, top, eff, window = {"s": (1024, 4096, 8, 2, 32, 4, 512, 1024), "m": (2048, 8192, 16, 4, 64, 4, 1024, 2048)}[size]
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top, "scale": 2.0}}
    delta = {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "conv": 4}}
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "conv": 4, "scale": 128 ** -0.5, "mask": {"size": window},
                     "rot": {"base": 10000.0, "dims": 64}}}
    return {"architecture": "Kipedra", "vocab": 32768, "width": D, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "kv_page_size": 16,
            "layers": [dict(delta, mlp={"kind": "dense", "ff": ff}), att, dict(att), dict(delta, mlp=moe)],
            "loop": {"start": 0, "stop": 4, "times": 2}}


def flint_routed_config(size):
    """The closest existing model at equal size: Flint with a window on every layer, two dense layers and six with routed
    experts: the same width, heads, window, experts (count, choice, width), vocabulary and number of executed layers."""
    D, ff, heads, kv, E, top, eff, window = {"s": (1024, 4096, 8, 2, 32, 4, 512, 1024), "m": (2048, 8192, 16, 4, 64, 4, 1024, 2048)}[size]
    return {"architectures": ["FlintForCausalLM"], "hidden_size": D, "num_hidden_layers": 8, "num_attention_heads": heads,
            "num_key_value_heads": kv, "head_dim": 128, "vocab_size": 32768, "n_routed_experts": E, "num_experts_per_tok": top,
            "moe_intermediate_size": eff, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "first_k_dense_replace": 2,
            "intermediate_size": ff, "kv_page_size": 16, "scoring_func": "sigmoid", "sliding_window": window,
            "sliding_window_pattern": [True] * 8}


def sigusun_config(size):
    """Sigusun at layer sizes that resemble a real model's: a retention layer, a latent attention layer in a sliding window, a
    second one that reads the first one's cached latent, and a causal latent attention layer with sinks; every layer with
    clamped routed experts, a shared expert and the per-layer token input; eight layers (the four kinds twice)."""
    D, heads, rank, E, top, eff, window = {"s": (1024, 8, 256, 32, 4, 512, 1024), "m": (2048, 16, 512, 64, 4, 1024, 2048)}[size]
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": E, "top": top}, "shared": {"ff": eff, "limit": 7.0}}
    latent = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": rank, "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
    ret = {"type": "retention", "mlp": moe,
           "mixer": {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5.0 - 5.0 * h / heads) for h in range(heads)],
                     "rot": {"base": 10000.0, "dims": 128}}}
    win = {"type": "latent_attention", "mlp": moe, "mixer": dict(latent, mask={"size": window})}
    sink = {"type": "latent_attention_2", "mlp": moe, "mixer": dict(latent)}
    layers = []
    for rep in range(2):
        at = len(layers)
        layers += [ret, win, dict(win, mixer=dict(win["mixer"], kv_from=at + 1)), sink]
    return {"architecture": "Sigusun", "vocab": 32768, "width": D, "norm": {"eps": 1e-6}, "token_side": {"dim": 64}, "kv_page_size": 16,
            "layers": layers}


def kitodra_config(size):
    """Kitodra at layer sizes that resemble a real model's: a lightning layer, a window layer whose values are its keys,
    a difference attention layer inside chunks (two maps of half a head's width) and another lightning layer, each with
    clamped routed experts chosen among the best groups and a shared expert; the four run twice, the second time as layers
    that use the first four's tensors (own caches and states); the token-pair table on the embedding."""
    D, heads, kv, E, top, eff, window = {"s": (1024, 8, 2, 32, 4, 512, 1024), "m": (2048, 16, 4, 64, 4, 1024, 2048)}[size]
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": E, "top": top, "groups": {"count": 8, "keep": 4}},
           "shared": {"ff": eff, "limit": 7.0}}
    light = {"type": "lightning", "mlp": moe,
             "mixer": {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5.0 - 5.0 * h / heads) for h in range(heads)]}}
    win = {"type": "attention_2", "mlp": moe, "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                         "mask": {"size": window}, "rot": {"base": 10000.0, "dims": 64}}}
    diff = {"type": "attention", "mlp": moe, "mixer": {"heads": heads, "kv_heads": kv, "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "softcap": 30.0,
                                                        "diff": 0.4, "mask": {"size": window}}}
    layers = [light, win, diff, dict(light)]
    layers += [dict(L, weights_of=i) for i, L in enumerate(layers)]
    return {"architecture": "Kitodra", "vocab": 32768, "width": D, "norm": {"eps": 1e-6}, "kv_page_size": 16,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers}


DESIGNS = {"pedotar": (("pedotar", pedotar_config), ("flint_dense", flint_dense_config)),
           "kitodra": (("kitodra", kitodra_config), ("sigusun", sigusun_config), ("kipedra", kipedra_config)),
           "kipedra": (("kipedra", kipedra_config), ("flint_routed", flint_routed_config)),
           "sigusun": (("sigusun", sigusun_config), ("kipedra", kipedra_config), ("pedotar", pedotar_config))}


def design_compare(args):
    """Prefill and decode throughput of another design beside the closest Flint model at equal layer sizes (random
    weights), and where each model's eager steps spend their time, launcher by launcher.  One JSON line."""
    import torch
    from quench6k_b200 import ops
    from quench6k_b200.config.registry import get_architecture
    from quench6k_b200.engine import ModelRunner, StepEntry
    pk = peaks()
    B, ctx, T, page = args.batch or 8, args.context or 4096, args.prefill_tokens, 16
    gen = torch.Generator().manual_seed(1)
    out = {"design": args.design, "dtype": args.dtype, "batch": B, "context": ctx, "prefill_tokens": T, "steps": args.steps,
           "warmup": args.warmup, "peaks": pk["source"], "sizes": {}}
    for size in [x for x in args.sizes.split(",") if x]:
        row = {}
        for name, make in DESIGNS[args.design]:
            cfg_d = make(size)
            arch = get_architecture(cfg_d.get("architecture") or cfg_d["architectures"][0])
            cfg = arch.config_cls.from_dict(cfg_d)
            pages = B * ((ctx + args.steps + args.warmup + 64) // page + 2) + T // page + 2
            runner = ModelRunner.from_random(cfg, 0, dtype=args.dtype, page_size=page, num_pages=pages, max_requests=B + 1, arch=arch)
            V = runner.vocab_size
            ids = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()

            def timed(fn, n, warm):
                for i in range(warm):
                    fn(i)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(warm, warm + n):
                    fn(i)
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1) / n

            # prefill: one prompt of T tokens in one step, a new request every time
            def prefill(i):
                runner.add_request(("p", i))
                runner.step([StepEntry(("p", i), ids(T), [T - 1])])
                runner.end_request(("p", i))
            ms_p = timed(prefill, max(3, args.steps // 4), 3)
            ops.profile_begin()
            prefill(10 ** 6)
            prof_p = ops.profile_end()
            # decode: B requests brought to the context by real prefill steps (the recurrent states are then real too)
            rids = [("d", j) for j in range(B)]
            for r in rids:
                runner.add_request(r)
                for at in range(0, ctx, T):
                    runner.step([StepEntry(r, ids(min(T, ctx - at)), [])])
            toks = [ids(args.steps + args.warmup + 8) for _ in rids]
            ms_d = timed(lambda i: runner.step([StepEntry(r, [toks[j][i]], [0]) for j, r in enumerate(rids)]), args.steps, args.warmup)
            runner.cuda_graphs = False
            ops.profile_begin()
            runner.step([StepEntry(r, [toks[j][-1]], [0]) for j, r in enumerate(rids)])
            prof_d = ops.profile_end()
            assert ops.tc_status() == 0
            table = lambda rec: sorted(({"op": tag, "launcher": fn, "calls": calls, "us": round(ms * 1e3, 1)} for (tag, fn), (calls, ms) in rec.items()),
                                       key=lambda x: -x["us"])
            row[name] = {"prefill_tok_s": round(T / ms_p * 1e3), "prefill_ms": round(ms_p, 3), "decode_tok_s": round(B / ms_d * 1e3),
                         "decode_ms": round(ms_d, 3), "graph_replays": runner.graph_replays,
                         "prefill_kernels": table(prof_p), "decode_kernels": table(prof_d)}
            del runner
            torch.cuda.empty_cache()
        out["sizes"][size] = row
    print(json.dumps(out))
    return 0


def workload_stress(args, shape):
    """A long prompt beside many short sampled requests, through the engine's own scheduler and
    paged cache: one request of `--context` (131,072) uniform-random tokens, greedy, 128 new tokens;
    `--batch - 1` (63) requests of 256 to 16,384 tokens at temperature 1.0, 128 new tokens each.
    Host wall clock around Engine.step() until everything has finished; one JSON line."""
    import torch
    from quench6k_b200 import Engine, SamplingParams, ops
    from quench6k_b200.config import FlintConfig
    torch.cuda.set_device(0)
    long_len, n_req, new = args.context or 131072, args.batch or 64, 128
    cfg_d = dict(CONFIG2)
    layers = args.layers or shape["layers"]
    cfg_d["num_hidden_layers"] = layers
    if args.page_size:
        cfg_d["kv_page_size"] = args.page_size
    cfg = FlintConfig.from_dict(cfg_d)
    page, budget = cfg.kv_page_size, args.prefill_tokens
    gen = torch.Generator().manual_seed(4)
    lens = [long_len] + [int(x) for x in torch.randint(256, min(16384, long_len) + 1, (n_req - 1,), generator=gen)]
    num_pages = sum((n + new + page - 1) // page + 1 for n in lens)      # every request fits at once: no preemption is forced
    t0 = time.time()
    eng = Engine.from_random(cfg, seed=0, dtype=args.dtype, page_size=page, num_pages=num_pages, max_requests=n_req,
                             max_batch_tokens=budget)
    torch.cuda.synchronize()
    print(f"[bench] model and cache ready in {time.time() - t0:.1f}s ({torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device)",
          file=sys.stderr, flush=True)
    V = cfg.vocab_size
    ids = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()
    warm = eng.generate([ids(budget), ids(300)], SamplingParams(max_tokens=4, temperature=0.0))      # first-call costs stay outside
    assert all(len(o.tokens) == 4 for o in warm)
    torch.cuda.synchronize()
    base = dict(eng.stats)
    clocks = ClockSampler()
    clocks.start()
    t1 = time.perf_counter()
    rids = [eng.add_request(ids(n), SamplingParams(max_tokens=new, temperature=0.0 if i == 0 else 1.0, seed=100 + i), rid=f"s{i}")
            for i, n in enumerate(lens)]
    done, first_long, decode_only_s, decode_only_tokens, last = {}, None, 0.0, 0, t1
    while len(done) < len(rids):
        prompts_left = any(not r.output for r in list(eng.scheduler.running) + list(eng.scheduler.waiting))
        tokens_before = eng.stats["tokens"]
        for out in eng.step():
            done[out.rid] = out
        now = time.perf_counter()
        if not prompts_left:                      # a step of decode tokens only
            decode_only_s += now - last
            decode_only_tokens += eng.stats["tokens"] - tokens_before
        if first_long is None and any(r.rid == "s0" and r.output for r in eng.scheduler.running):
            first_long = now - t1
        last = now
    torch.cuda.synchronize()
    total_s = time.perf_counter() - t1
    clock_info = clocks.stop()
    assert ops.tc_status() == 0
    generated = sum(len(o.tokens) for o in done.values())
    print(json.dumps({
        "workload": "stress: a long greedy prompt in portions beside sampled requests, continuous batching", "impl": "ours",
        "config": {"model": shape["label"], "layers": layers, "layers_full": shape["layers"], "requests": n_req, "long_prompt": long_len,
                   "other_prompts": "uniform 256..16384", "new_tokens": new, "token_budget": budget, "page_size": page,
                   "pages": num_pages, "dtype": args.dtype},
        "prompt_tokens": sum(lens), "generated_tokens": generated, "seconds": round(total_s, 3),
        "tokens_per_s": round((sum(lens) + generated) / total_s, 1),
        "long_prompt_first_token_s": None if first_long is None else round(first_long, 3),
        "decode_only": {"tokens": decode_only_tokens, "tok_per_s": round(decode_only_tokens / decode_only_s, 1) if decode_only_s else None},
        "steps": eng.stats["steps"] - base["steps"], "preemptions": eng.stats["preemptions"] - base["preemptions"],
        "gib_on_device": round(torch.cuda.max_memory_allocated() / 2**30, 1), "clocks": clock_info}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--config", type=int, default=2, choices=sorted(SHAPES),
                    help="2: 24 layers at 32,768 cached tokens (the default run); 3: the full 48 layers at 8,192 cached tokens")
    ap.add_argument("--workload", default="decode", choices=["decode", "stress"],
                    help="stress: one 131,072-token prompt in 2,048-token portions and 128 decoded tokens beside 63 sampled requests "
                         "of 256 to 16,384 tokens, all through Engine.step() (its own JSON line; --context and --batch scale it down)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64", help="further decode batch sizes, comma separated ('' for none)")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature of the end-to-end part (0: greedy, the headline)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--page-size", type=int, default=None, help="KV page size (default: the configuration's 16)")
    ap.add_argument("--profile-ops", action="store_true",
                    help="instead of the benchmark line: where an eager decode step and a prefill step spend their time, launcher by "
                         "launcher (CUDA events around every launch; its own JSON line)")
    ap.add_argument("--design", default=None, choices=["pedotar", "kipedra", "sigusun", "kitodra"],
                    help="instead of the benchmark line: prefill and decode throughput of that design beside the closest Flint model "
                         "(pedotar: dense feed-forwards; kipedra: windows and routed experts; sigusun: beside Kipedra and Pedotar; kitodra: beside Sigusun and Kipedra) at equal layer sizes (--sizes), with each "
                         "model's time launcher by launcher (its own JSON line)")
    ap.add_argument("--sizes", default="s,m", help="--design: s (width 1024) and/or m (width 2048)")
    ap.add_argument("--kernel", default=None, choices=["attention_prefill", "gated_delta", "retention"],
                    help="time one kernel alone at the configuration's head sizes instead of the model: attention_prefill runs "
                         "--prefill-tokens query tokens that end at position --context (one request, contiguous pages); gated_delta runs "
                         "the delta rule recurrence over one portion of --prefill-tokens tokens, or with --batch over that many single tokens; "
                         "retention does the same for the retention recurrence")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "lkarlslund/quench6k is a Rust workspace (Cargo.toml, no setup.py or "
                          "pyproject.toml): pip cannot install it offline, cargo/rustc are absent, and its kernels are sm_120a-only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from quench6k_b200 import Engine, SamplingParams, ops
    from quench6k_b200.config import FlintConfig
    from quench6k_b200.engine import StepEntry

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    if args.kernel == "attention_prefill":
        return kernel_attention_prefill(args)
    if args.kernel == "gated_delta":
        return kernel_gated_delta(args)
    if args.kernel == "retention":
        return kernel_retention(args)
    if args.design:
        torch.cuda.set_device(0)
        return design_compare(args)
    torch.cuda.set_device(0)
    pk = peaks()
    shape = SHAPES[args.config]
    if args.workload == "stress":
        return workload_stress(args, shape)
    args.batch = args.batch or 8
    args.context = args.context or shape["context"]
    cfg_d = dict(CONFIG2)
    full_layers = shape["layers"]
    layers = args.layers or full_layers
    cfg_d["num_hidden_layers"] = layers
    if args.page_size:
        cfg_d["kv_page_size"] = args.page_size
    cfg = FlintConfig.from_dict(cfg_d)
    page = cfg.kv_page_size
    point_batches = [int(x) for x in args.points.split(",") if x.strip()]
    max_b = max([args.batch] + point_batches)
    ctx = args.context
    headroom = max(96, args.steps + args.warmup + 16)            # every timed request decodes that many tokens past its context
    pages_per_req = (ctx + headroom + page - 1) // page + 1
    num_pages = max(max_b * pages_per_req, (args.prefill_tokens + page - 1) // page + 1)
    t0 = time.time()
    eng = Engine.from_random(cfg, seed=0, dtype=args.dtype, page_size=page, num_pages=num_pages, max_requests=max_b,
                             max_batch_tokens=max(args.prefill_tokens, max_b))
    runner = eng.runner
    for c in runner.caches:                      # stand-in for the keys and values a prefill would have left
        c.k.normal_(0.0, 0.5)
        c.v.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    print(f"[bench] model and cache ready in {time.time() - t0:.1f}s ({torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device)",
          file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(1)
    V = cfg.vocab_size

    def rand_ids(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    def stand_at_context(rids):
        for r in rids:
            runner.add_request(r)
        chunk = args.prefill_tokens              # pages are taken as a chunked prefill would take them:
        for at in range(0, ctx, chunk):          # one portion of each request in turn
            for r in rids:
                runner.assume_cached(r, min(chunk, ctx - at))

    def graphs_equal_eager(B, n=64, prompt=4096):
        """The reference times nothing before it has checked it (crates/cli/src/flint.rs:116-131: 64 graph-decoded
        tokens must equal eager decoding): B prompts are prefilled in portions, then n greedy tokens are decoded by
        replaying CUDA graphs; the same again with eager launches; the ids must be equal.  (Real prompts, not the
        random cache contents of the timed part: those differ from page to page, and the two passes get other pages.)"""
        prompt = min(prompt, ctx)
        prompts = [rand_ids(prompt) for _ in range(B)]
        seqs = []
        for graphs in (True, False):
            rids = [f"g{B}_{i}" for i in range(B)]
            keep, runner.cuda_graphs = runner.cuda_graphs, runner.cuda_graphs and graphs
            cur = []
            for r, toks in zip(rids, prompts):
                runner.add_request(r)
                for at in range(0, prompt, args.prefill_tokens):
                    part = toks[at:at + args.prefill_tokens]
                    logits = runner.step([StepEntry(r, part, [len(part) - 1])])
                cur.append(int(ops.argmax(logits)[0]))
            ids = [cur]
            for _ in range(n):
                cur = ops.argmax(runner.step([StepEntry(r, [cur[j]], [0]) for j, r in enumerate(rids)])).tolist()
                ids.append(cur)
            runner.cuda_graphs = keep
            for r in rids:
                runner.end_request(r)
            seqs.append(ids)
        return seqs[0] == seqs[1], len({t for step in seqs[0] for t in step})

    def experts_read(one, first, B, n=2):
        """Distinct experts per routed layer that n further (eager) decode steps really chose, on average."""
        from quench6k_b200.parts.base import Tap
        tap = Tap(max(64, B))
        routed = [b.ffn for b in runner.model.blocks if hasattr(b.ffn, "routing_tap")]
        for f in routed:
            f.routing_tap = tap
        keep, runner.cuda_graphs = runner.cuda_graphs, False
        total, count = 0, 0
        for i in range(first, first + n):
            one(i)
            for (what, _), buf in tap.buffers.items():
                if what == "experts":
                    total += int(torch.unique(buf[:B]).numel())
                    count += 1
        runner.cuda_graphs = keep
        for f in routed:
            f.routing_tap = None
        return total / count if count else None

    def timed_decode(B, steps, warmup, sampler=None):
        """Device-timed decode steps of B requests standing at `ctx` cached tokens: (ms per step, launches, distinct
        experts per layer the router chose in two further steps)."""
        rids = [f"d{B}_{i}" for i in range(B)]
        stand_at_context(rids)
        toks = [rand_ids(steps + warmup + 2) for _ in rids]

        def one(i):
            logits = runner.step([StepEntry(r, [toks[j][i]], [0]) for j, r in enumerate(rids)])
            return ops.argmax(logits)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        l0 = ops.launch_count
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.start()                      # the clocks are read while the timed steps run, and only then
        a.record()
        for i in range(warmup, warmup + steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        if sampler is not None:
            sampler.result = sampler.stop()
        ms = a.elapsed_time(b) / steps
        launches = ops.launch_count - l0
        chosen = experts_read(one, warmup + steps, B)
        for r in rids:
            runner.end_request(r)
        return ms, launches, chosen

    if args.profile_ops:
        return profile_ops(args, runner, cfg_d, layers, ctx, stand_at_context, rand_ids)
    checked, distinct = graphs_equal_eager(args.batch)
    if not checked:
        print("bench.py: decoding by CUDA-graph replay and by eager launches gave different tokens; nothing is timed", file=sys.stderr)
        return 1
    clocks = ClockSampler()
    ms, launches, chosen = timed_decode(args.batch, args.steps, args.warmup, clocks)
    clock_info = clocks.result
    value = args.batch * 1000.0 / ms
    total_b, w_b, kv_b = decode_bytes(cfg_d, layers, args.batch, ctx, chosen)
    achieved = total_b / (ms * 1e-3) / 1e9

    # prefill: one prompt of T tokens in one step, the logits of its last token wanted
    T = args.prefill_tokens
    pre_ms = []
    for it in range(3):
        runner.add_request("p")
        ids = rand_ids(T)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([StepEntry("p", ids, [T - 1])])
        b.record()
        torch.cuda.synchronize()
        pre_ms.append(a.elapsed_time(b))
        runner.end_request("p")
    pms = min(pre_ms[1:])
    pf = prefill_flops(cfg_d, layers, T)
    pb = prefill_bytes(cfg_d, layers, T)
    prefill = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
               "frac": round(pf / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               # a step of milliseconds runs under the power cap: the sustained product rate is its yardstick; and the step
               # cannot be shorter than its weights take to stream, nor than that plus its products one after the other
               "frac_sustained": round(pf / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
               "bytes_floor_ms": round(pb / pk["hbm_gbs"] / 1e6, 3),
               "flops_floor_ms": round(pf / pk["bf16_tflops_sustained"] / 1e9, 3)}

    # end to end: Engine.step() with host ids in and sampled ids out each step
    for i in range(args.batch):
        sp = SamplingParams(max_tokens=args.steps + args.warmup + 8, temperature=args.temperature, seed=1000 + i)
        eng.adopt_request(rand_ids(ctx), rand_ids(1)[0], sp)
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(args.steps):
        eng.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    for r in list(eng.scheduler.running):
        eng.abort(r.rid)
    R = args.batch
    h2d = 4 * (3 * R + (R + 1) + 2 * R + R + R * ((ctx + 64 + page - 1) // page))       # the step's int32 block, tables included
    e2e = {"value": round(args.batch * args.steps / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4 * R}
    if args.temperature > 0:
        e2e["temperature"] = args.temperature
        e2e["h2d_bytes_per_step"] += 32 * R               # the rows' sampling records

    # further batch sizes last: their long steps at batch 64 warm the GPU up, which the headline numbers should not feel
    points, points_roofline, points_ms = {}, {}, {}
    for B in point_batches:
        bms, _, bchosen = timed_decode(B, args.steps, 3)
        points[f"decode_b{B}"] = round(B * 1000.0 / bms, 1)
        points_ms[f"decode_b{B}"] = round(bms, 3)
        points_roofline[f"decode_b{B}"] = round(decode_bytes(cfg_d, layers, B, ctx, bchosen)[0] / (bms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    out = {
        "metric": f"decode tok/s at batch {args.batch} (context {ctx}); prefill tok/s at {T} tokens; % of roofline",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype in ("bfloat16", "bf16") else "fp32",
        "data": "synthetic: seeded random weights N(0,0.02), uniform-random token ids, caches filled with random values",
        "config": {"model": shape["label"], "layers": layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "experts": cfg.n_routed_experts, "top_k": cfg.num_experts_per_tok,
                   "expert_width": cfg.moe_intermediate_size, "vocab": cfg.vocab_size, "rope_theta": cfg.rope_theta,
                   "page_size": page, "global_batch": args.batch, "seq_len": ctx, "prefill_tokens": T,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights and cache stream from HBM every step)",
                   "kv_fill": "random values; pages taken in portions of prefill_tokens per request in turn", "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes": int(total_b), "weight_bytes": int(w_b), "kv_bytes": int(kv_b),
                     "experts_read_per_layer": None if chosen is None else round(chosen, 1)},
        "points": points, "points_roofline": points_roofline, "points_ms": points_ms,
        "checked": {"graph_replay_equals_eager": True, "tokens": 64, "distinct_ids": distinct},
        "e2e": e2e, "gpu_launches": launches, "clocks": clock_info, "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
