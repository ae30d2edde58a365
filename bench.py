#!/usr/bin/env python3
"""Decode and prefill throughput of wick_b200 on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--model 8b|14b|32b]
    python bench.py --design nibotar|tuguvik|fasunex|sunosun [--design-size 2k|4k]      (a line of its own, see below)

The default run has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32
heads over 8 kv heads of 128, intermediate 12288, vocabulary 151936) with random
bfloat16 weights drawn on the device, a batch of 8 sequences with 512-token
random-id prompts, and a context of 4096 tokens per sequence.  A "step" is one
decode step of the whole batch.

``value``: decoded tokens per second, timed on the device with CUDA events over
exactly K steps after W warm-up steps, as the median of three such regions
(``spread`` has the fastest and the slowest); ``e2e``: the same through the Python
entry point ``wick_b200.generate``, token ids going in and coming out on the host.
``prefill``: one 2,048-token prompt (median of 40 steps back to back, about a second).  ``roofline``: the bytes a
decode step has to read (every weight it uses once, plus the cache of the live
requests) over its time, against the measured copy bandwidth.  ``points``: decode
at batch 1 and 64, and the workloads at Qwen3-14B sizes (ragged batch of 16,
prompts of 64 to 2,048 tokens) and Qwen3-32B sizes (batch 8, 1,024-token prompts),
each with its fraction of the copy bandwidth.  Every weight matrix is far larger
than the L2 cache, so consecutive steps never find their inputs there.  The run
fails if any step it timed produced logits that are not finite.

``--design nibotar`` leaves the default workload alone and prints another line: prefill
(one 2,048-token prompt) and decode (batch 8 and 64, 512-token prompts) throughput of the
Nibotar design at layer sizes that resemble a real model's (random weights), beside Qwen3
at equal size (same width, heads, layers and vocabulary; its intermediate size is what a
Nibotar token's experts and shared expert add up to), and ``parts``: where a prompt step and
a decode step of each spend their time, per kind of kernel, with the fraction of the
measured peak each reaches (a second process times them with CUDA events around every call,
launched one by one without programmatic dependent launch, so that they do not overlap).
``--design tuguvik`` does the same for the Tuguvik design (layers of differential attention
and of attention through a cached latent, every layer with a gated feed-forward of Qwen3's
intermediate size and a token input); its ``parts`` count each kernel's own arithmetic and
bytes, so that every kind can be held against the measured peaks.
``--design fasunex`` prints the line of the Fasunex design (layers that alternate between a chunked attention beside a
state-space recurrence and an attention whose keys are its values, routed experts with identity outputs) beside Nibotar,
the closest design here, at equal size, with the same kind of ``parts``.
``--design sunosun`` prints the line of the Sunosun design (layers that alternate between a softmax attention beside a gated
linear attention and a gated linear attention alone; one-matrix experts chosen within groups, with a gated shared expert)
beside Fasunex, the closest design here (its parallel mixer holds a state-space recurrence with a state of the same size),
at equal size, with the same kind of ``parts``; the recurrences' scans are also held against the float32 rate of the CUDA
cores, since that, not memory, bounds them in a prompt.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

def _qwen3(hidden, heads, kv_heads, intermediate, layers):
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=hidden, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=128, intermediate_size=intermediate, num_hidden_layers=layers,
                vocab_size=151936, max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False)


# The layer sizes of the three Qwen3 models measured here, and their workloads:
# 8b: batch 1 / 8 / 64, 512-token prompts (the headline is batch 8) and one 2,048-token prompt;
# 14b: a ragged batch of 16, prompt lengths uniform in [64, 2048] in one prompt step, 128 decode steps;
# 32b: a batch of 8 with 1,024-token prompts, 128 decode steps.
MODELS = {"8b": _qwen3(4096, 32, 8, 12288, 36), "14b": _qwen3(5120, 40, 8, 17408, 40),
          "32b": _qwen3(5120, 64, 8, 25600, 64)}
QWEN3_8B = MODELS["8b"]
CONTEXT = 4096
PROMPT = 512
PREFILL = 2048
REPEATS = 3
E2E_WARMUP = 24
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            j = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(j.get(k), (int, float)):
                out[k] = float(j[k])
        out["source"] = "measured"
        return out
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while it is open."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass
        return self

    def __exit__(self, *a):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                           "samples": len(sm)}


def reference_arm():
    # wick is a Rust program (Cargo.toml, no Python package): pip cannot build it
    # and this image has no cargo/rustc.
    print(json.dumps({"impl": "reference",
                      "unavailable": "pMag11-alt/wick is a Rust crate without a Python package; no cargo/rustc "
                                     "in this image, so it cannot be installed or run offline"}))
    return 0


def device_timed_decode(torch, wick, eng, prompts, steps, warmup, repeats=REPEATS):
    """The prompts in one step, W decode steps, then ``repeats`` timed regions of exactly
    ``steps`` decode steps each (CUDA events on the launching stream, a synchronize on both
    sides).  The batch is stepped the way ``wick_b200.generate`` steps it: the sampled token
    and the lengths stay on the device, the host launches a step ahead and reads every step's
    tokens from pinned memory one step behind.  Returns the regions' milliseconds per step, the
    kernels launched in one region, the cached tokens a step reads on average, the prompt
    step's milliseconds, and whether the last step's logits were finite."""
    from wick_b200 import ops
    batch = len(prompts)
    slots = [eng.open_seq() for _ in prompts]
    total = warmup + repeats * steps + 2
    for s, p in zip(slots, prompts):
        eng.cache.reserve(s, len(p) + total)
    run = eng.begin_run(wick.SamplerConfig.greedy(), ())
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run.start(slots, prompts, [1 << 30] * batch)
    e1.record()
    run.collect()
    prompt_ms = e0.elapsed_time(e1)
    for _ in range(warmup):
        run.launch(slots)
        run.collect()
    regions, launches, kv_tokens = [], 0, 0.0
    for _ in range(repeats):
        torch.cuda.synchronize()
        l0 = ops.launches[0]
        kv_tokens = sum(eng.seq_len(s) for s in slots) + batch * (steps + 1) / 2.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            run.launch(slots)
            if k:
                run.collect()
        e1.record()
        run.collect()
        torch.cuda.synchronize()
        regions.append(e0.elapsed_time(e1) / steps)
        launches = ops.launches[0] - l0
    finite = run.last_logits is not None and bool(torch.isfinite(run.last_logits).all().item())
    eng.check_kernels()
    for s in slots:
        eng.close_seq(s)
    return regions, launches, kv_tokens, prompt_ms, finite


def decode_point(torch, wick, eng, pk, prompts, steps, warmup, repeats=REPEATS):
    """One decode workload as a dictionary: tokens a second (median region), spread, roofline."""
    regions, launches, kv_tokens, prompt_ms, finite = device_timed_decode(torch, wick, eng, prompts, steps, warmup, repeats)
    ms = statistics.median(regions)
    step_bytes = eng.model.weight_bytes_per_step() + eng.cache.read_bytes(int(kv_tokens), len(prompts))
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {"value": len(prompts) * 1e3 / ms, "ms_per_step": ms, "ms_min": min(regions), "ms_max": max(regions),
            "regions": len(regions), "gb_per_step": step_bytes / 1e9, "hbm_frac": achieved / pk["hbm_gbs"],
            "achieved_gbs": achieved, "launches": launches, "prompt_ms": prompt_ms, "finite": finite}


def random_prompts(torch, vocab, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lens]


def other_model(torch, wick, pk, name, steps, warmup, layers=None):
    """The 14b / 32b workload on an engine of its own (built here, dropped afterwards)."""
    cfg_json = dict(MODELS[name])
    full = cfg_json["num_hidden_layers"]
    if layers:
        cfg_json["num_hidden_layers"] = min(layers, full)
    cfg = wick.config_from_json(cfg_json)
    if name == "14b":
        g = torch.Generator().manual_seed(14)
        lens = torch.randint(64, 2049, (16,), generator=g).tolist()
    else:
        lens = [1024] * 8
    need = sum((n + warmup + REPEATS * steps + 2 + 63) // 64 * 64 for n in lens)
    t0 = time.time()
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=need)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    out = decode_point(torch, wick, eng, pk, random_prompts(torch, cfg.vocab_size, lens, 15), steps, warmup)
    out.update({"layers": len(eng.spec.schedule), "layers_of_config": full, "batch": len(lens),
                "prompt_tokens": sum(lens), "load_s": load_s,
                "prompt_tok_s": sum(lens) / (out["prompt_ms"] * 1e-3)})
    del eng
    torch.cuda.empty_cache()
    return out


# Layer sizes for --design: Nibotar (one dense layer, then layers of experts) and Qwen3 at equal size.
DESIGN_SIZES = {
    "2k": dict(width=2048, heads=16, kv=4, dim=128, layers=8, vocab=32768, mask=1024, dense_ff=8192, experts=8, top=2,
               expert_ff=1536, shared_ff=2048),
    "4k": dict(width=4096, heads=32, kv=8, dim=128, layers=4, vocab=32768, mask=2048, dense_ff=16384, experts=16, top=2,
               expert_ff=2048, shared_ff=4096),
}


def design_configs(z):
    mixer = dict(heads=z["heads"], kv_heads=z["kv"], dim=z["dim"], vdim=z["dim"], scale=z["dim"] ** -0.5, v_mix=True,
                 mask={"size": z["mask"]}, rot={"dims": z["dim"], "base": 1000000.0})
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    layers = [dict(type="attention", mixer=mixer, mlp={"kind": "dense", "ff": z["dense_ff"]} if i == 0 else moe)
              for i in range(z["layers"])]
    nib = dict(architecture="Nibotar", vocab=z["vocab"], width=z["width"], norm={"eps": 1e-5}, postln_alpha=2.0,
               logit_softcap=30.0, layers=layers)
    qwen = _qwen3(z["width"], z["heads"], z["kv"], z["top"] * z["expert_ff"] + z["shared_ff"], z["layers"])
    qwen.update(head_dim=z["dim"], vocab_size=z["vocab"])
    return {"nibotar": nib, "qwen3": qwen}


def design_step_bytes(eng, z, name, batch, kv_tokens):
    """Bytes a decode step has to read: every weight it uses once, plus the cache it reads.  Of a layer's experts a
    batch uses E (1 - (1 - top / E)^batch) on average; a block mask reads at most one block of positions."""
    n = eng.model.weight_bytes_per_step()
    if name == "nibotar":
        e, top = z["experts"], z["top"]
        one = 3 * z["expert_ff"] * z["width"] * 2
        used = e * (1.0 - (1.0 - top / e) ** batch)
        n += (z["layers"] - 1) * (used - top) * one
        kv_tokens = min(kv_tokens, batch * z["mask"])
    if name == "tuguvik":
        kv_tokens = min(kv_tokens, batch * (z["window"] + z["keep_first"]))
    if name == "fasunex":
        return fasunex_step_bytes(eng, z, batch, kv_tokens)
    if name == "sunosun":
        return sunosun_step_bytes(eng, z, batch, kv_tokens)
    return n + eng.cache.read_bytes(int(kv_tokens), batch)


def design_model(torch, wick, pk, z, name, cfg_json, steps, warmup):
    cfg = wick.config_from_json(cfg_json)
    per_seq = (PROMPT + warmup + REPEATS * steps + 2 + 64 + 63) // 64 * 64
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max(64 * per_seq, PREFILL + 64))
    out = {}
    ptoks = random_prompts(torch, z["vocab"], [PREFILL], 3)[0]
    times = []
    for i in range(3 + 10):
        s = eng.open_seq()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = eng.step([s], [ptoks])
        e1.record()
        torch.cuda.synchronize()
        eng.close_seq(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    ok = bool(torch.isfinite(logits).all().item())
    pms = statistics.median(times)
    out["prefill"] = {"tokens": PREFILL, "ms": pms, "tok_s": PREFILL / (pms * 1e-3)}
    for b in (8, 64):
        regions, launches, kv_tokens, _, finite = device_timed_decode(
            torch, wick, eng, random_prompts(torch, z["vocab"], [PROMPT] * b, 10 + b), steps, warmup)
        ms = statistics.median(regions)
        nbytes = design_step_bytes(eng, z, name, b, kv_tokens)
        out[f"decode_b{b}"] = {"tok_s": b * 1e3 / ms, "ms_per_step": ms, "gb_per_step": nbytes / 1e9,
                               "hbm_frac": nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], "launches": launches}
        ok = ok and finite
    out["finite"] = ok
    del eng
    torch.cuda.empty_cache()
    return out


def design_parts(torch, wick, pk, z, name, cfg_json):
    """Microseconds per layer that a 2,048-token prompt step and a decode step of 8 sequences (1,500 cached positions
    each) spend in each kind of kernel, with what each reaches of the measured peak."""
    from wick_b200 import ops
    cfg = wick.config_from_json(cfg_json)
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=8 * 1600 + PREFILL + 64, use_graphs=False)
    acc = {}

    def timed(kind, fn):
        def run(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(torch.cuda.current_stream())
            r = fn(*a, **kw)
            e1.record(torch.cuda.current_stream())
            acc.setdefault(kind, []).append((e0, e1))
            return r
        return run

    for fname, kind in (("attention_masked", "attention"), ("attention_prompt", "attention"),
                        ("attention_decode_parts_fused", "attention+finish"), ("attention_decode", "attention"),
                        ("qkv_finish", "finish"), ("qk_norm_rope_append", "finish"), ("scaled_add_rmsnorm", "norm"),
                        ("rmsnorm", "norm")):
        setattr(ops, fname, timed(kind, getattr(ops, fname)))       # (the parts call these through the module)
    for blk in eng.model.blocks:
        blk.ffn.forward = timed("ffn " + type(blk.ffn).__name__, blk.ffn.forward)
        m = blk.mixer
        m.qkv.forward_delta = timed("qkv product", m.qkv.forward_delta)
        m.o.forward_delta = timed("o product", m.o.forward_delta)
    L, D, H, G, d = z["layers"], z["width"], z["heads"], z["kv"], z["dim"]
    act_ff = z["top"] * z["expert_ff"] + z["shared_ff"]

    def collect(n_tok, kv_read_tokens, att_pairs):
        torch.cuda.synchronize()
        res = {}
        for kind, evs in acc.items():
            res[kind] = {"us_per_layer": sum(a.elapsed_time(b) for a, b in evs) * 1e3 / L}
        acc.clear()
        qkv_w, o_w = D * (H + 2 * G) * d, D * H * d
        for kind, r in res.items():
            t = r["us_per_layer"] * 1e-6
            if kind in ("qkv product", "o product"):
                w = qkv_w if kind[0] == "q" else o_w
                r["tflops"], r["gbs"] = 2.0 * n_tok * w / t / 1e12, 2.0 * w / t / 1e9
            elif kind.startswith("ffn"):
                if "MLP" in kind and "Gated" not in kind:
                    w = 2 * D * z["dense_ff"]
                    r["us_per_layer"] *= L                     # (one such layer)
                    t *= L
                elif "TableMoE" in kind:
                    w = 3 * D * act_ff
                    r["us_per_layer"] *= L / (L - 1.0)
                    t *= L / (L - 1.0)
                else:
                    w = 3 * D * act_ff
                r["tflops"] = 2.0 * n_tok * w / t / 1e12
            elif kind.startswith("attention"):
                r["tflops"] = 4.0 * H * d * att_pairs / t / 1e12
                r["gbs"] = kv_read_tokens * 2 * G * d * 2 / t / 1e9
            elif kind == "norm":
                r["gbs"] = n_tok * D * (4 + 4 + 4 + 2) / (t / 2) / 1e9      # two norms a layer; stream in, sums in, stream out, copy out
            elif kind == "finish":
                r["gbs"] = n_tok * (H + 2 * G) * d * (4 + 2) / t / 1e9
            for k, peak in (("tflops", pk["bf16_tflops"]), ("gbs", pk["hbm_gbs"])):
                if k in r:
                    r[k + "_frac"] = r[k] / peak
        return res

    out = {}
    ptoks = random_prompts(torch, z["vocab"], [PREFILL], 3)[0]
    for i in range(3):
        s = eng.open_seq()
        acc.clear()
        eng.step([s], [ptoks])
        eng.close_seq(s)
    n = PREFILL
    blk = z["mask"] if name == "nibotar" else None
    pairs = sum((p % blk if blk else p) + 1 for p in range(n))
    out["prompt_2048"] = collect(n, n, pairs)
    slots = [eng.open_seq() for _ in range(8)]
    ctx = random_prompts(torch, z["vocab"], [1500] * 8, 4)
    eng.step(slots, ctx)
    for i in range(4):
        acc.clear()
        eng.step(slots, [[1 + i]] * 8)
    seen = (min(1504, 1504 % blk + 1) if blk else 1504)
    out["decode_b8_ctx1500"] = collect(8, 8 * seen, 8 * seen)
    return out


def design_compare(args) -> int:
    import torch
    import wick_b200 as wick
    pk = peaks()
    z = DESIGN_SIZES[args.design_size]
    cfgs = design_configs(z)
    if args.design_parts:
        print(json.dumps({name: design_parts(torch, wick, pk, z, name, cfgs[name]) for name in ("nibotar", "qwen3")}))
        return 0
    steps, warmup = min(args.steps, 64), max(args.warmup, 3)
    with Clocks() as clk:
        models = {name: design_model(torch, wick, pk, z, name, cfgs[name], steps, warmup) for name in ("nibotar", "qwen3")}
    env = dict(os.environ, WICK_B200_NO_PDL="1")
    r = subprocess.run([sys.executable, os.path.abspath(__file__), "--design", args.design, "--design-size", args.design_size,
                        "--design-parts"], env=env, capture_output=True, text=True)
    parts = None
    for ln in r.stdout.splitlines():
        if ln.startswith("{"):
            parts = json.loads(ln)
    line = {"metric": f"Nibotar beside Qwen3 at equal size ({args.design_size}): prefill and decode tok/s, bf16", "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "sizes": z,
            "data": "synthetic: seeded random weights, seeded uniform random token ids", "models": models, "parts": parts,
            "parts_error": None if parts is not None else r.stderr[-600:], "clocks": clk.result, "peaks": pk}
    print(json.dumps(line))
    return 0 if all(m["finite"] for m in models.values()) else 1


# ---- --design tuguvik ----------------------------------------------------------
# Layer sizes: differential attention with as many numbers a head as Qwen3 (two maps of 64), attention through a latent
# of 512 + 64 numbers a position with heads of 128 + 64 query numbers and 128 values; windows; a gated feed-forward.
TUGUVIK_SIZES = {
    "2k": dict(width=2048, heads=16, kv=4, dim=128, layers=8, vocab=32768, window=1024, keep_first=4, ff=5120, q_rank=768,
               kv_rank=512, rot_dim=64, side=256),
    "4k": dict(width=4096, heads=32, kv=8, dim=128, layers=4, vocab=32768, window=2048, keep_first=4, ff=10240, q_rank=1536,
               kv_rank=512, rot_dim=64, side=256),
}


def tuguvik_configs(z):
    d = z["dim"]
    diff = dict(heads=z["heads"], kv_heads=z["kv"], dim=d // 2, vdim=d, scale=(d // 2) ** -0.5, diff=0.8,
                mask={"size": z["window"], "keep_first": z["keep_first"]},
                rot={"dims": d // 2, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})

    def latent(src):
        m = dict(heads=z["heads"], dim=d, rot_dim=z["rot_dim"], vdim=d, q_rank=z["q_rank"], kv_rank=z["kv_rank"],
                 scale=(d + z["rot_dim"]) ** -0.5, mask={"size": z["window"]},
                 rot={"dims": z["rot_dim"], "base": 10000.0, "scaling": {"factor": 40.0, "fast": 32.0, "slow": 1.0, "original": 4096}})
        if src is not None:
            m["kv_from"] = src
        return m
    layers = []
    for i in range(z["layers"]):                      # differential, latent, latent on the same rows, differential, ...
        kind = (0, 1, 2, 0)[i % 4]
        mixer = diff if kind == 0 else latent(None if kind == 1 else i - 1)
        layers.append(dict(type="attention" if kind == 0 else "latent_attention", mixer=mixer, mlp={"kind": "dense", "ff": z["ff"]}))
    tug = dict(architecture="Tuguvik", vocab=z["vocab"], width=z["width"], norm={"eps": 1e-5}, token_side={"dim": z["side"]},
               layers=layers)
    qwen = _qwen3(z["width"], z["heads"], z["kv"], z["ff"], z["layers"])
    qwen.update(head_dim=d, vocab_size=z["vocab"])
    return {"tuguvik": tug, "qwen3": qwen}


def tuguvik_parts(torch, wick, pk, z, name, cfg_json):
    """What a 2,048-token prompt step and a decode step of 8 sequences (1,500 cached positions each) spend in each kind of
    kernel: microseconds a step (all layers), and the kernels' own arithmetic and bytes over that time against the measured
    peaks.  Every call of a kernel's Python face is timed with CUDA events and says what it computes and moves."""
    from wick_b200 import ops
    from wick_b200.parts.linear import Linear
    cfg = wick.config_from_json(cfg_json)
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=8 * 1600 + PREFILL + 64, use_graphs=False)
    acc = {}
    ctx = {"pairs": 0, "kv_rows": 0}

    def timed(kind, fn, work):
        def run(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(torch.cuda.current_stream())
            r = fn(*a, **kw)
            e1.record(torch.cuda.current_stream())
            acc.setdefault(kind, []).append((e0, e1) + tuple(work(r, *a, **kw)))
            return r
        return run

    def nbytes(*ts):
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def product(kind, lin):
        w = lin.out_features * lin.in_features
        n_out = lin.out_features // 2 if lin.gated else lin.out_features
        for fname in ("forward", "forward_delta"):
            setattr(lin, fname, timed(kind, getattr(lin, fname),
                                      lambda r, x, *a, **k: (2.0 * x.shape[0] * w, 2 * w + nbytes(x) + (nbytes(r) if r is not None else 4 * x.shape[0] * n_out))))

    # attention: a pair of a query and a visible key costs, per head, the score and the weighted sum of every map
    def attn_multi_work(r, q, store, batch, scale, **kw):
        n, H, d = q.shape
        e = kw["v_dim"]
        return 2.0 * ctx["pairs"] * H * (d + kw["maps"] * e), nbytes(q, r) + ctx["kv_rows"] * store[0].numel() // 64 * store.element_size()

    def attn_flex_work(r, q, k0, k1, v, batch, scale, **kw):
        n, heads, dk = q.shape
        row_bytes = 2 * (k0[8] + k1[8] + v[8]) * (heads if not k0[9] else 1)      # (flat sources hold every head's rows)
        return 2.0 * ctx["pairs"] * heads * (dk + kw["dv"]), nbytes(q, r) + ctx["kv_rows"] * row_bytes

    def attn_std_work(r, q, kv, batch, *a, **k):
        n, H, d = q.shape
        return 4.0 * ctx["pairs"] * H * d, nbytes(q, r) + ctx["kv_rows"] * kv[0].numel() // 64 * kv.element_size()

    def rows_work(r, *a, **k):
        ts = [t for t in a if torch.is_tensor(t)] + [t for t in k.values() if torch.is_tensor(t) and t.dim() >= 2 and t.numel() < (1 << 26)]
        out = [t for t in (r if isinstance(r, tuple) else (r,)) if torch.is_tensor(t)]
        return 0.0, nbytes(*[t for t in ts if t.numel() < (1 << 26)], *out)

    def absorb_work(r, parts, uk, H, d, dr, rank, **k):
        return 2.0 * parts.shape[1] * H * d * rank, nbytes(parts, uk, r)

    def expand_work(r, y, uv, gate, H, e, rank, **k):
        return 2.0 * y.shape[0] * H * e * rank, nbytes(y, uv, r)

    def norm_work(r, x, delta=None, *a, **k):
        return 0.0, nbytes(x, delta) + (nbytes(x) if delta is not None and k.get("rows") is None else 0) + (nbytes(r) if r is not None and r is not x else 0)

    for fname, kind, work in (("attention_multi", "attention", attn_multi_work), ("attention_flex", "attention", attn_flex_work),
                              ("combine_maps", "attention", rows_work), ("latent_query", "finish", rows_work),
                              ("attention_prompt", "attention", attn_std_work),
                              ("attention_decode", "attention", attn_std_work), ("qkv_finish", "finish", rows_work),
                              ("latent_finish", "finish", rows_work), ("qk_norm_rope_append", "finish", rows_work),
                              ("latent_absorb", "query into the rows' space", absorb_work),
                              ("latent_expand", "values out of the rows' space", expand_work), ("stream_update", "norm", norm_work),
                              ("rmsnorm", "norm", lambda r, x, *a, **k: norm_work(r, x, k.get("delta"), rows=k.get("rows"))),
                              ("gelu_gate_rows", "side input", rows_work)):
        setattr(ops, fname, timed(kind, getattr(ops, fname), work))       # (the parts call these through the module)
    # (the fused decode attention of the standard mixer would hide its parts: the plain sequence of kernels is timed instead)
    ops.attention_decode_parts_supported = lambda *a, **k: False
    for blk in eng.model.blocks:
        m = blk.mixer
        for attr, kind in (("qkv", "projections into the mixer"), ("down", "projections into the mixer"),
                           ("uq", "projections into the mixer"), ("ukv", "keys and values from the latent"), ("o", "o product")):
            if isinstance(getattr(m, attr, None), Linear):
                product(kind, getattr(m, attr))
        for attr in ("gate_up", "down"):
            product("feed-forward", getattr(blk.ffn, attr))
        if blk.side is not None:
            product("side input", blk.side.gate)
            product("side input", blk.side.proj)

    def collect():
        torch.cuda.synchronize()
        res = {}
        for kind, evs in acc.items():
            us = sum(e[0].elapsed_time(e[1]) for e in evs) * 1e3
            fl, by = sum(e[2] for e in evs), sum(e[3] for e in evs)
            r = res[kind] = {"us_per_step": us, "calls": len(evs)}
            if fl and kind.startswith("recurrence ("):
                r["fp32_tflops"] = fl / (us * 1e-6) / 1e12
                r["fp32_frac_of_nominal"] = r["fp32_tflops"] / FP32_TFLOPS_NOMINAL
            elif fl:
                r["tflops"] = fl / (us * 1e-6) / 1e12
                r["tflops_frac"] = r["tflops"] / pk["bf16_tflops"]
            r["gbs"] = by / (us * 1e-6) / 1e9
            r["gbs_frac"] = r["gbs"] / pk["hbm_gbs"]
        acc.clear()
        return res

    out = {}
    win, keep = (z["window"], z["keep_first"]) if name == "tuguvik" else (None, 0)
    seen = lambda p: p + 1 if win is None else min(p + 1, win + (keep if name == "tuguvik" else 0))   # (an upper bound for kept keys)
    ptoks = random_prompts(torch, z["vocab"], [PREFILL], 3)[0]
    ctx["pairs"], ctx["kv_rows"] = sum(seen(p) for p in range(PREFILL)), PREFILL
    for i in range(3):
        s = eng.open_seq()
        acc.clear()
        eng.step([s], [ptoks])
        eng.close_seq(s)
    out["prompt_2048"] = collect()
    slots = [eng.open_seq() for _ in range(8)]
    eng.step(slots, random_prompts(torch, z["vocab"], [1500] * 8, 4))
    ctx["pairs"] = ctx["kv_rows"] = 8 * seen(1503)
    for i in range(4):
        acc.clear()
        eng.step(slots, [[1 + i]] * 8)
    out["decode_b8_ctx1500"] = collect()
    return out


def tuguvik_compare(args) -> int:
    import torch
    import wick_b200 as wick
    pk = peaks()
    z = TUGUVIK_SIZES[args.design_size]
    cfgs = tuguvik_configs(z)
    if args.design_parts:
        print(json.dumps({args.design_parts: tuguvik_parts(torch, wick, pk, z, args.design_parts, cfgs[args.design_parts])}))
        return 0
    steps, warmup = min(args.steps, 64), max(args.warmup, 3)
    with Clocks() as clk:
        models = {name: design_model(torch, wick, pk, z, name, cfgs[name], steps, warmup) for name in ("tuguvik", "qwen3")}
    env = dict(os.environ, WICK_B200_NO_PDL="1")
    parts, errors = {}, {}
    for name in ("tuguvik", "qwen3"):                  # (a process each: the timing wrappers replace the module's functions)
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--design", "tuguvik", "--design-size", args.design_size,
                            "--design-parts", name], env=env, capture_output=True, text=True)
        for ln in r.stdout.splitlines():
            if ln.startswith("{"):
                parts.update(json.loads(ln))
        if name not in parts:
            errors[name] = r.stderr[-600:]
    line = {"metric": f"Tuguvik beside Qwen3 at equal size ({args.design_size}): prefill and decode tok/s, bf16", "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "sizes": z,
            "data": "synthetic: seeded random weights, seeded uniform random token ids", "models": models, "parts": parts,
            "parts_error": errors or None, "clocks": clk.result, "peaks": pk}
    print(json.dumps(line))
    return 0 if all(m["finite"] for m in models.values()) else 1


# ---- --design fasunex ----------------------------------------------------------
# Fasunex beside Nibotar, the closest design here (attention over blocks of positions with a sink, experts): the same width,
# heads, layers, vocabulary, block size and experts.  Layers alternate between the parallel mixer (chunked attention beside
# a state-space recurrence of `ssm_heads` x `ssm_dim` numbers with a state of `ssm_state`) and the attention whose keys are
# its values; every layer has routed experts with two identity outputs.
FP32_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12      # 148 SMs x 128 lanes x one multiply-add a cycle at 1965 MHz


def fasunex_configs(z):
    d = z["dim"]
    left = dict(heads=z["heads"], kv_heads=z["kv"], dim=d, vdim=d, scale=d ** -0.5, mask={"size": z["mask"]},
                rot={"dims": d // 2, "base": 10000.0})
    right = dict(heads=z["width"] // 64, vdim=64, state=128, groups=2, conv=4, norm_groups=2)
    att = dict(heads=z["heads"], kv_heads=z["kv"], dim=d, vdim=d, scale=d ** -0.5)
    mlp = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "identity": 2, "top": z["top"]}}
    layers = [dict(type="parallel", mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0), mlp=mlp) if i % 2 == 0
              else dict(type="attention", mixer=att, mlp=mlp) for i in range(z["layers"])]
    fas = dict(architecture="Fasunex", vocab=z["vocab"], width=z["width"], norm={"eps": 1e-5}, layers=layers)
    return {"fasunex": fas, "nibotar": design_configs(z)["nibotar"]}


def fasunex_step_bytes(eng, z, batch, kv_tokens):
    """Bytes a decode step of Fasunex has to read: the weights (of a layer's experts a batch uses E (1 - (1 - top / (E + I))^batch)
    on average), the keys and values (a chunked layer reads at most one chunk a sequence) and the recurrences' records."""
    n = eng.model.weight_bytes_per_step()
    e, top, outs = z["experts"], z["top"], z["experts"] + 2
    one = 3 * z["expert_ff"] * z["width"] * 2
    n += z["layers"] * (e * (1.0 - (1.0 - top / outs) ** batch) - min(top, e)) * one
    row = 2 * z["kv"] * z["dim"] * 2
    half = z["layers"] // 2
    n += (z["layers"] - half) * min(kv_tokens, batch * z["mask"]) * row + half * kv_tokens * row
    for g in eng.cache.groups:
        if g.need.kind == "state":
            n += 2 * g.store.read_bytes(0, batch)                  # (read and written back)
    return n


def fasunex_parts(torch, wick, pk, z, name, cfg_json):
    """What a 2,048-token prompt step and a decode step of 8 sequences (1,500 cached positions each) spend in each kind of
    kernel: microseconds a step (all layers), and the kernels' own arithmetic and bytes over that time against the measured
    peaks (tensor-core peak for the matrix products and the attention, copy bandwidth for the rest)."""
    from wick_b200 import ops
    from wick_b200.parts.linear import Linear
    cfg = wick.config_from_json(cfg_json)
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=8 * 1600 + PREFILL + 64, max_seqs=16, use_graphs=False)
    acc = {}
    ctx = {"pairs": 0, "kv_rows": 0, "blocked": True}

    def timed(kind, fn, work):
        def run(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(torch.cuda.current_stream())
            r = fn(*a, **kw)
            e1.record(torch.cuda.current_stream())
            acc.setdefault(kind, []).append((e0, e1) + tuple(work(r, *a, **kw)))
            return r
        return run

    def nbytes(*ts):
        return sum(t.numel() * t.element_size() for t in ts if torch.is_tensor(t))

    def product(kind, lin):
        w = lin.out_features * lin.in_features
        for fname in ("forward", "forward_delta"):
            setattr(lin, fname, timed(kind, getattr(lin, fname),
                                      lambda r, x, *a, **k: (2.0 * x.shape[0] * w, 2 * w + nbytes(x) + (nbytes(r) if r is not None else 4 * x.shape[0] * lin.out_features))))

    def attn_work(r, q, kv, batch, scale, **kw):
        n, H, d = q.shape
        blocked = kw.get("mask", "causal") == "block"
        pairs, rows = (ctx["pairs_block"], ctx["rows_block"]) if blocked else (ctx["pairs"], ctx["kv_rows"])
        return 4.0 * pairs * H * d, nbytes(q, r) + rows * kv[0].numel() // 64 * kv.element_size()

    def rows_work(r, *a, **k):
        ts = [t for t in a if torch.is_tensor(t)] + [t for t in k.values() if torch.is_tensor(t) and t.dim() >= 2]
        out = [t for t in (r if isinstance(r, tuple) else (r,)) if torch.is_tensor(t)]
        return 0.0, nbytes(*[t for t in ts if t.numel() < (1 << 27)], *[t for t in out if not any(t is x for x in ts)])

    def ssm_work(r, parts, **k):
        n = parts.shape[1]
        H, Pn, N = k["heads"], k["head_dim"], k["state"]
        ch = H * Pn + 2 * k["groups"] * N
        rec = 2 * 4 * k["batch"].n_seqs * (H * Pn * N + (k["taps"] - 1) * ch)
        # (two multiply-adds per number of the state and token: the update and the read-out)
        return 4.0 * n * H * Pn * N, nbytes(parts) + 4 * n * (2 * ch + H * Pn) + rec

    def gla_work(r, parts, **k):
        n = parts.shape[1]
        H, dk, dv = k["heads"], k["key_dim"], k["v_dim"]
        rec = 2 * 4 * k["batch"].n_seqs * H * dk * dv
        return 4.0 * n * H * dk * dv, nbytes(parts, r) + 2 * 4 * n * (3 * H * dk + H * dv) + rec

    def norm_work(r, x, delta=None, *a, **k):
        return 0.0, nbytes(x, delta) + (nbytes(x) if delta is not None and k.get("rows") is None else 0) + (nbytes(r) if r is not None and r is not x else 0)

    def ffn_work(width, ff, top, share, shared_ff, mats=3, shared_mats=3):
        def work(r, x, *a, **k):
            n = x.shape[0]
            act = mats * top * share * ff + shared_mats * shared_ff
            return (2.0 * n * width * act,
                    nbytes(x, r) + min(n * top, z["experts"]) * mats * width * ff * 2 + shared_mats * width * shared_ff * 2)
        return work

    for fname, kind, work in (("attention_masked", "attention", attn_work), ("qkv_finish", "finish", rows_work),
                              ("gate_rows_", "output gate", rows_work), ("ssm_mix", "recurrence (convolution, scan)", ssm_work),
                              ("ssm_gate_norm", "recurrence's gate and norm", rows_work), ("weighted_sum", "sum of the branches", rows_work),
                              ("gla_mix", "recurrence (decays, scan)", gla_work), ("gla_norm_gate", "recurrence's gate and norm", rows_work),
                              ("embed_sinusoid", "embedding", rows_work),
                              ("concat_activation", "pass input", rows_work), ("stream_update", "norm", norm_work),
                              ("scaled_add_rmsnorm", "norm", lambda r, x, delta, *a, **k: norm_work(r, x, delta)),
                              ("rmsnorm", "norm", lambda r, x, *a, **k: norm_work(r, x, k.get("delta"), rows=k.get("rows")))):
        setattr(ops, fname, timed(kind, getattr(ops, fname), work))       # (the parts call these through the module)
    W = z["width"]
    for blk in eng.model.blocks:
        mixers = getattr(blk.mixer, "branches", [blk.mixer])
        for m in mixers:
            for attr, kind in (("qkv", "projections into the mixer"), ("input", "projections into the mixer"), ("o", "o product")):
                if isinstance(getattr(m, attr, None), Linear):
                    product(kind, getattr(m, attr))
        f = blk.ffn
        if type(f).__name__ == "RoutedMoE":
            sh = f.shared.intermediate if f.shared is not None else 0
            work = ffn_work(W, f.intermediate, f.top, f.experts / float(f.outputs), sh, 3 if f.gated else 2, 2)
        elif type(f).__name__ == "TableMoE":
            work = ffn_work(W, f.intermediate, f.top, 1.0, z["shared_ff"])
        else:
            work = ffn_work(W, z["dense_ff"], 1, 1.0, 0)
        f.forward = timed("feed-forward " + type(f).__name__, f.forward, work)

    def collect():
        torch.cuda.synchronize()
        res = {}
        for kind, evs in acc.items():
            us = sum(e[0].elapsed_time(e[1]) for e in evs) * 1e3
            fl, by = sum(e[2] for e in evs), sum(e[3] for e in evs)
            r = res[kind] = {"us_per_step": us, "calls": len(evs)}
            if fl and kind.startswith("recurrence ("):
                r["fp32_tflops"] = fl / (us * 1e-6) / 1e12
                r["fp32_frac_of_nominal"] = r["fp32_tflops"] / FP32_TFLOPS_NOMINAL
            elif fl:
                r["tflops"] = fl / (us * 1e-6) / 1e12
                r["tflops_frac"] = r["tflops"] / pk["bf16_tflops"]
            r["gbs"] = by / (us * 1e-6) / 1e9
            r["gbs_frac"] = r["gbs"] / pk["hbm_gbs"]
        acc.clear()
        return res

    out = {}
    blk = z["mask"]
    ptoks = random_prompts(torch, z["vocab"], [PREFILL], 3)[0]
    ctx["pairs"], ctx["kv_rows"] = sum(p + 1 for p in range(PREFILL)), PREFILL
    ctx["pairs_block"], ctx["rows_block"] = sum(p % blk + 1 for p in range(PREFILL)), PREFILL
    for i in range(3):
        s = eng.open_seq()
        acc.clear()
        eng.step([s], [ptoks])
        eng.close_seq(s)
    out["prompt_2048"] = collect()
    slots = [eng.open_seq() for _ in range(8)]
    eng.step(slots, random_prompts(torch, z["vocab"], [1500] * 8, 4))
    ctx["pairs"] = ctx["kv_rows"] = 8 * 1504
    ctx["pairs_block"] = ctx["rows_block"] = 8 * (1503 % blk + 1)
    for i in range(4):
        acc.clear()
        eng.step(slots, [[1 + i]] * 8)
    out["decode_b8_ctx1500"] = collect()
    return out


def fasunex_compare(args) -> int:
    import torch
    import wick_b200 as wick
    pk = peaks()
    z = DESIGN_SIZES[args.design_size]
    cfgs = fasunex_configs(z)
    if args.design_parts:
        print(json.dumps({args.design_parts: fasunex_parts(torch, wick, pk, z, args.design_parts, cfgs[args.design_parts])}))
        return 0
    steps, warmup = min(args.steps, 64), max(args.warmup, 3)
    with Clocks() as clk:
        models = {name: design_model(torch, wick, pk, z, name, cfgs[name], steps, warmup) for name in ("fasunex", "nibotar")}
    env = dict(os.environ, WICK_B200_NO_PDL="1")
    parts, errors = {}, {}
    for name in ("fasunex", "nibotar"):                # (a process each: the timing wrappers replace the module's functions)
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--design", "fasunex", "--design-size", args.design_size,
                            "--design-parts", name], env=env, capture_output=True, text=True)
        for ln in r.stdout.splitlines():
            if ln.startswith("{"):
                parts.update(json.loads(ln))
        if name not in parts:
            errors[name] = r.stderr[-600:]
    line = {"metric": f"Fasunex beside Nibotar at equal size ({args.design_size}): prefill and decode tok/s, bf16", "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "sizes": z,
            "data": "synthetic: seeded random weights, seeded uniform random token ids", "models": models, "parts": parts,
            "parts_error": errors or None, "clocks": clk.result, "peaks": pk}
    print(json.dumps(line))
    return 0 if all(m["finite"] for m in models.values()) else 1


# ---- --design sunosun ----------------------------------------------------------
# Sunosun beside Fasunex, the closest design here (a softmax attention beside a recurrence in one mixer, routed experts): the
# same width, heads, layers, vocabulary and experts.  Layers alternate between the parallel mixer (attention with biases and a
# sink of score 0 beside a gated linear attention of width / 128 heads with 128 key channels and 128 values, a state as large as
# Fasunex's recurrence) and a gated linear attention alone.  The experts have two matrices where Fasunex's have three, so
# their inner size is half as large again; every layer has the shared expert.
def sunosun_configs(z):
    d = z["dim"]
    left = dict(heads=z["heads"], kv_heads=z["kv"], dim=d, vdim=d, scale=d ** -0.5)
    right = dict(heads=z["width"] // 128, dim=128, vdim=128, tau=16.0)
    mlp = {"kind": "moe", "expert": {"ff": z["expert_ff"] * 3 // 2}, "shared": {"ff": z["shared_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    layers = [dict(type="parallel", mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0), mlp=mlp) if i % 2 == 0
              else dict(type="gla", mixer=right, mlp=mlp) for i in range(z["layers"])]
    suno = dict(architecture="Sunosun", vocab=z["vocab"], width=z["width"], norm={"eps": 1e-5}, embedding={"scale": 1.0},
                logit_softcap=30.0, layers=layers)
    return {"sunosun": suno, "fasunex": fasunex_configs(z)["fasunex"]}


def sunosun_step_bytes(eng, z, batch, kv_tokens):
    """Bytes a decode step of Sunosun has to read: the weights (of a layer's experts a batch uses E (1 - (1 - top / E)^batch)
    on average), the keys and values of the layers that have an attention, and the recurrences' records (read and written)."""
    n = eng.model.weight_bytes_per_step()
    e, top = z["experts"], z["top"]
    one = 2 * (z["expert_ff"] * 3 // 2) * z["width"] * 2
    n += z["layers"] * (e * (1.0 - (1.0 - top / e) ** batch) - min(top, e)) * one
    n += (z["layers"] - z["layers"] // 2) * kv_tokens * 2 * z["kv"] * z["dim"] * 2
    for g in eng.cache.groups:
        if g.need.kind == "state":
            n += 2 * g.store.read_bytes(0, batch)
    return n


def sunosun_compare(args) -> int:
    import torch
    import wick_b200 as wick
    pk = peaks()
    z = DESIGN_SIZES[args.design_size]
    cfgs = sunosun_configs(z)
    if args.design_parts:
        print(json.dumps({args.design_parts: fasunex_parts(torch, wick, pk, z, args.design_parts, cfgs[args.design_parts])}))
        return 0
    steps, warmup = min(args.steps, 64), max(args.warmup, 3)
    with Clocks() as clk:
        models = {name: design_model(torch, wick, pk, z, name, cfgs[name], steps, warmup) for name in ("sunosun", "fasunex")}
    env = dict(os.environ, WICK_B200_NO_PDL="1")
    parts, errors = {}, {}
    for name in ("sunosun", "fasunex"):                # (a process each: the timing wrappers replace the module's functions)
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--design", "sunosun", "--design-size", args.design_size,
                            "--design-parts", name], env=env, capture_output=True, text=True)
        for ln in r.stdout.splitlines():
            if ln.startswith("{"):
                parts.update(json.loads(ln))
        if name not in parts:
            errors[name] = r.stderr[-600:]
    line = {"metric": f"Sunosun beside Fasunex at equal size ({args.design_size}): prefill and decode tok/s, bf16", "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "sizes": z,
            "data": "synthetic: seeded random weights, seeded uniform random token ids", "models": models, "parts": parts,
            "parts_error": errors or None, "clocks": clk.result, "peaks": pk, "fp32_tflops_nominal": FP32_TFLOPS_NOMINAL}
    print(json.dumps(line))
    return 0 if all(m["finite"] for m in models.values()) else 1


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8b", choices=sorted(MODELS), help="8b: the headline line with all its parts; "
                    "14b / 32b: only that model's workload, as a line of its own")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the timed decode steps")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL, help="tokens of the prefill step (the default workload's is 2,048)")
    ap.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of --steps decode steps each (median reported)")
    ap.add_argument("--skip-points", action="store_true", help="no batch 1 / 64 runs")
    ap.add_argument("--skip-models", action="store_true", help="no 14b / 32b workloads")
    ap.add_argument("--skip-e2e", action="store_true", help="no run through the Python entry point")
    ap.add_argument("--prefill-steps", type=int, default=0, help="timed prompt steps (default: about a second's worth, at most 40)")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-decode", action="store_true", help="prefill only (for profiling)")
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs (every kernel is a launch of its own)")
    ap.add_argument("--design", default=None, choices=["nibotar", "tuguvik", "fasunex", "sunosun"],
                    help="another line: this design beside Qwen3 (fasunex: beside Nibotar; sunosun: beside Fasunex) at equal size")
    ap.add_argument("--design-size", default="2k", choices=sorted(DESIGN_SIZES))
    ap.add_argument("--design-parts", nargs="?", const="both", default=None,
                    help="only the per-kernel times of --design (run by --design itself; tuguvik: of the model named)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.design == "tuguvik":
        return tuguvik_compare(args)
    if args.design == "fasunex":
        return fasunex_compare(args)
    if args.design == "sunosun":
        return sunosun_compare(args)
    if args.design:
        return design_compare(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)
    repeats = max(1, args.repeats)
    steps = max(1, min(args.steps, (CONTEXT - args.prompt_len - max(warmup, E2E_WARMUP) - 2) // repeats))

    import torch

    import wick_b200 as wick
    from wick_b200 import ops

    pk = peaks()
    if args.model != "8b":
        with Clocks() as clk:
            out = other_model(torch, wick, pk, args.model, steps, warmup, args.layers)
        out.update({"metric": f"Qwen3-{args.model.upper()} sizes bf16 decode tok/s", "unit": "tokens/s", "clocks": clk.result,
                    "peaks": pk["source"]})
        print(json.dumps(out))
        return 0
    cfg_json = dict(QWEN3_8B)
    full_layers = cfg_json["num_hidden_layers"]
    if args.layers:
        cfg_json["num_hidden_layers"] = args.layers
    cfg = wick.config_from_json(cfg_json)
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    per_seq = (args.prompt_len + warmup + repeats * steps + 2 + 64 + 63) // 64 * 64
    n_prefill = args.prefill_tokens
    max_tokens = max(max_batch * per_seq, n_prefill + 64)
    t0 = time.time()
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens,
                                  use_graphs=False if args.eager else None)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    vocab = cfg.vocab_size

    # ---- decode, device-timed (the headline value) ----
    with Clocks() as clk:
        if args.skip_decode:
            head = {"value": float("nan"), "ms_per_step": float("nan"), "launches": 0, "achieved_gbs": float("nan"),
                    "hbm_frac": float("nan"), "gb_per_step": float("nan"), "finite": True, "ms_min": None, "ms_max": None}
        else:
            head = decode_point(torch, wick, eng, pk, random_prompts(torch, vocab, [args.prompt_len] * args.batch, 1),
                                steps, warmup, repeats)
    ms = head["ms_per_step"]

    # ---- decode through the Python entry point, host tokens in and out ----
    # One generate() call per region: the prompts, E2E_WARMUP untimed decode steps (the steps
    # right after a prompt step run up to 15 % slower for some 20 steps while the clocks
    # recover from the prompt's power draw; the device-timed regions leave them out through
    # their warm-up steps too), then exactly K steps timed on the host's clock between the
    # loop's per-step callbacks.  Every step's ids reach the host before its callback runs.
    e2e_value, e2e_whole, h2d, d2h = None, None, None, None
    e2e_warmup = max(warmup, E2E_WARMUP)
    prompts = random_prompts(torch, vocab, [args.prompt_len] * args.batch, 2)
    opts = wick.GenOptions(max_tokens=1 + e2e_warmup + steps, sampler=wick.SamplerConfig.greedy(), context=CONTEXT,
                           max_batch=args.batch)
    if not args.skip_e2e and not args.skip_decode:
        wick.generate(eng, [p[:16] for p in prompts], wick.GenOptions(max_tokens=4, sampler=wick.SamplerConfig.greedy(),
                                                                      context=CONTEXT, max_batch=args.batch))
        runs = []
        begin = eng.begin_run
        eng.begin_run = lambda *a, **kw: runs.append(begin(*a, **kw)) or runs[-1]
        vals, whole = [], []
        for _ in range(repeats):
            stamps = []
            res = wick.generate(eng, prompts, opts, on_step=lambda n, live: stamps.append(time.perf_counter()))
            assert len(stamps) == 1 + e2e_warmup + steps and all(len(r.tokens) == 1 + e2e_warmup + steps for r in res)
            vals.append(args.batch * steps / (stamps[-1] - stamps[e2e_warmup]))
            whole.append(sum(len(r.tokens) - 1 for r in res) / (max(r.gen_ms for r in res) * 1e-3))
        del eng.begin_run
        e2e_value, e2e_whole = statistics.median(vals), statistics.median(whole)
        # what crosses the bus: the prompts' description once, a description of the decode batch
        # when its composition changes, and the sampled ids (with a status word) every step
        h2d = sum(r.h2d_bytes for r in runs) / (repeats * (1 + e2e_warmup + steps))
        d2h = (args.batch + 1) * 4

    # ---- prefill of one 2,048-token prompt ----
    ptoks = random_prompts(torch, vocab, [n_prefill], 3)[0]
    times = []
    # The fraction is of the peak SUSTAINED under the power cap (a seconds-long loop of products), so the prompt
    # step is timed in the same state: after 3 warm-up steps, a second or so of steps back to back (the first
    # steps of a product-heavy phase run at the part's full clock, the next ones while the power control settles).
    pf_warm = 3
    pf_timed = 0 if args.skip_prefill else (args.prefill_steps or max(5, min(40, int(40 * 2048 / max(n_prefill, 1)))))
    for i in range(0 if args.skip_prefill else pf_warm + pf_timed):
        s = eng.open_seq()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        plog = eng.step([s], [ptoks])
        e1.record()
        torch.cuda.synchronize()
        eng.close_seq(s)
        if i >= pf_warm:
            times.append(e0.elapsed_time(e1))
            head["finite"] = head["finite"] and bool(torch.isfinite(plog).all().item())
    pms = statistics.median(times) if times else float("nan")
    c = cfg
    gemm_params = len(eng.spec.schedule) * (c.hidden_size * (2 * c.q_dim + 2 * c.kv_dim) + 3 * c.hidden_size * c.intermediate_size)
    flops = 2.0 * n_prefill * gemm_params + 2.0 * vocab * c.hidden_size            # head on one row
    flops += len(eng.spec.schedule) * 4.0 * c.num_attention_heads * c.head_dim * n_prefill * (n_prefill + 1) / 2
    prefill = {"value": n_prefill / (pms * 1e-3), "tokens": n_prefill, "ms": pms,
               "frac": flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
               "tflops": flops / (pms * 1e-3) / 1e12, "peak_tflops": pk["bf16_tflops_sustained"],
               "ms_min": min(times) if times else None, "ms_max": max(times) if times else None, "timed_steps": len(times)}

    # ---- other batch sizes, other models ----
    points = {}
    if not args.skip_points and not args.skip_decode:
        for b in (1, 64):
            pt = decode_point(torch, wick, eng, pk, random_prompts(torch, vocab, [args.prompt_len] * b, 10 + b),
                              min(steps, 64), warmup, repeats)
            points[f"decode_b{b}"] = pt["value"]
            points[f"decode_b{b}_hbm_frac"] = pt["hbm_frac"]
            head["finite"] = head["finite"] and pt["finite"]
    n_layers = len(eng.spec.schedule)
    del eng
    torch.cuda.empty_cache()
    if not args.skip_models and not args.skip_decode and not args.layers:
        for name in ("14b", "32b"):
            pt = other_model(torch, wick, pk, name, min(steps, 128), warmup)
            points[f"qwen3_{name}_decode"] = pt["value"]
            points[f"qwen3_{name}_hbm_frac"] = pt["hbm_frac"]
            points[f"qwen3_{name}_ms_per_step"] = pt["ms_per_step"]
            points[f"qwen3_{name}_prompt_tok_s"] = pt["prompt_tok_s"]
            head["finite"] = head["finite"] and pt["finite"]
    if not head["finite"]:
        print("bench.py: a step produced logits that are not finite", file=sys.stderr)
        return 1

    line = {
        "metric": f"Qwen3-8B bf16 decode tok/s @ bs {args.batch} ({args.prompt_len}-token prompts, context {CONTEXT})",
        "value": head["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), seeded uniform random token ids",
        "config": {"model": "Qwen3-8B sizes", "layers": n_layers, "layers_of_config": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": args.prompt_len, "parallelism": "none",
                   "l2": "inputs larger than L2 (weights per step far exceed 126 MB)",
                   "peaks": pk["source"], "timed_regions": repeats,
                   "points_models": "qwen3_14b: 40 layers, ragged batch 16, prompts U[64,2048]; qwen3_32b: 64 layers, "
                                    "batch 8, 1024-token prompts; 128 decode steps each"},
        "spread": {"ms_min": head["ms_min"], "ms_max": head["ms_max"], "regions": repeats},
        "clocks": clk.result,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "warmup_steps": e2e_warmup, "from_first_token": e2e_whole,
                "note": "wick_b200.generate, host clock over the last K steps of each call; prompt ids and the batch "
                        "description go to the device when a batch starts or changes, every step's sampled ids "
                        "come back through pinned memory; from_first_token counts every decode step of the call"},
        "gpu_launches": head["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": head["achieved_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": head["hbm_frac"], "bytes_per_step": head["gb_per_step"] * 1e9},
        "points": points,
        "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
