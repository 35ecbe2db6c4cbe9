"""Decode and prefill throughput of the Llama-3.1-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 with every sequence at
the context length 8192 (one step = one decode step of the whole batch, timed with CUDA events
around K steps after W warm-up steps).  ``e2e`` is the same batch through the Python entry point
(``LlogosModel.generate``: host token ids in, host token ids out, sampling included): one call that
runs the eight prompts, 32 untimed decode steps and then the K timed ones, timed on the host clock
from the arrival of the tokens; ``whole_call_tokens_per_s`` is the rate over all decode steps of the call.
``prefill`` is one prompt of 2,048 tokens; ``roofline`` relates the decode step to the bytes it has
to read; ``points`` holds decode at batch 1 and 64.  Every step reads far more than the 126 MB of
L2 (16 GB of weights plus the cache), so no L2 flush is needed between steps.

``points`` also holds the three workloads the metric is quoted on, as they are written, each through the Python
entry point (prompts really run, every step sampled): ``llama8b_b8_ragged_to_8192`` (8 prompts of 128 to 2,048
tokens decoded until each holds 8,192), ``qwen3_8b_b16_256steps_greedy`` / ``..._t0.7`` (16 prompts of 64 to 4,096
tokens, 256 steps) and ``qwen25_14b_b32_128steps`` (32 prompts of 256 to 8,192 tokens, 128 greedy steps); each gives
decoded tokens per second over the whole run and the mean fraction of the copy bandwidth that the bytes of its decode
steps stand for.  The two workloads of a few hundred steps are run twice and the second run is the one reported (the first
records the CUDA graphs of its decode steps inside its decode time); the one of thousands of steps is run once.  ``--no-workloads`` leaves them out.
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

LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 131072,
    "attention_bias": False, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
# The other two shapes that the reference's numbers are quoted on; the default run keeps the first.
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "attention_bias": False, "tie_word_embeddings": False,
}
QWEN25_14B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 48, "hidden_size": 5120,
    "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 13824,
    "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 131072,
    "tie_word_embeddings": False,
}
# Further sizes of the same architecture, for looking at the kernels away from the headline shape (`--shape`): a
# small model with heads of 64 and tied embeddings, and the layer sizes of a 70B model (run with --layers 8 or so:
# all 80 layers do not fit beside a cache).
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 131072,
    "attention_bias": False, "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
LLAMA_70B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 80, "hidden_size": 8192,
    "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 28672,
    "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 131072,
    "attention_bias": False, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
SHAPES = {"llama-3.1-8b": ("Llama-3.1-8B shape", LLAMA_8B), "qwen3-8b": ("Qwen3-8B shape", QWEN3_8B),
          "qwen2.5-14b": ("Qwen2.5-14B shape", QWEN25_14B), "llama-3.2-1b": ("Llama-3.2-1B shape", LLAMA_1B),
          "llama-3.1-70b": ("Llama-3.1-70B shape", LLAMA_70B)}
CONTEXT = 8192
PREFILL_TOKENS = 2048


def pages_of(tokens):
    """Tokens that a request of so many tokens holds in the cache: whole pages of 64."""
    return -(-tokens // 64) * 64


def peaks():
    """Measured peaks from MEASURED_PEAKS.json beside this file when it exists, else an earlier measurement of a B200."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            if d.get("hbm_gbs") and d.get("bf16_tflops"):
                out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
                if d.get("bf16_tflops_sustained"):
                    out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        except (ValueError, OSError):
            pass
    return out


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg, n_layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i            # matrices only; norms are negligible
    return {"layer_params": per_layer, "matrix_params": per_layer * n_layers, "head_params": v * h,
            "kv_bytes_per_token": 2 * kv * 2 * n_layers}


def probe_decode_attention(torch, ops, shape, pk):
    """Decode attention alone with CUDA events: the cache contents are rotated through several layers' worth of pages
    so that L2 holds none of them.  One line per batch shape: bytes, time, rate, fraction of the copy bandwidth."""
    dev = "cuda:0"
    nh, nkv, hd = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    g = torch.Generator().manual_seed(0)
    cases = [("1 x 8192", [8192]), ("8 x 8192", [8192] * 8), ("64 x 8192", [8192] * 64), ("8 x 2048", [2048] * 8),
             ("8 x 32768", [32768] * 8), ("one of 8000, seven of 100", [8000] + [100] * 7),
             ("8, lengths 128..8192", [int(x) for x in torch.randint(128, 8192, (8,), generator=g)]),
             ("64, lengths 128..8192", [int(x) for x in torch.randint(128, 8192, (64,), generator=g)]),
             ("256 x 500", [500] * 256)]
    for label, lens in cases:
        b = len(lens)
        pages_per = [(n + 63) // 64 for n in lens]
        n_pages = sum(pages_per) + 1
        layer_bytes = n_pages * nkv * 64 * hd * 2 * 2
        layers = max(2, min(16, int(600e6 // layer_bytes) + 1))
        kps = [torch.randn(n_pages, nkv, 64, hd, device=dev).bfloat16() for _ in range(layers)]
        vps = [torch.randn(n_pages, nkv, 64, hd, device=dev).bfloat16() for _ in range(layers)]
        ring = max(pages_per)
        table = torch.zeros(b + 1, ring, dtype=torch.int32)
        p = 0
        for i in range(b):
            for j in range(pages_per[i]):
                table[i, j] = p
                p += 1
        table = table.to(dev)
        slots = torch.arange(b, dtype=torch.int32, device=dev)
        lb = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev)
        q = torch.randn(b, nh, hd, device=dev).bfloat16()
        out = torch.empty(b, nh * hd, device=dev, dtype=torch.bfloat16)
        nbytes = sum(lens) * nkv * hd * 2 * 2
        plan = ops.attn_decode_plan(torch.bfloat16, b, nh, nkv, hd, max(lens))
        scratch = torch.empty(max(1, plan.scratch_floats), device=dev)
        counters = torch.zeros(max(1, plan.n_counters), dtype=torch.int32, device=dev)

        def run(i):
            ops.attn_decode(q, kps[i % layers], vps[i % layers], table, ring, slots, lb, out, scratch,
                            scale=hd ** -0.5, window=0, plan=plan, counters=counters)
        for i in range(layers + 3):
            run(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(40):
            run(i)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / 40 * 1e3
        gbs = nbytes / us / 1e3
        print(f"decode attention ({plan.kind}) {label:28s} {nbytes / 1e6:8.1f} MB {us:8.1f} us {gbs:7.0f} GB/s "
              f"{gbs / pk['hbm_gbs']:.2f} of {pk['hbm_gbs']:.0f}", flush=True)
        del kps, vps
        torch.cuda.empty_cache()
    return 0


def probe_leave_one_out(torch, L, ops, cfg, batch, context):
    """The decode step of the whole model, recorded as a CUDA graph with one kernel left out at a time (the results are
    then meaningless; only the time is read): what each kernel costs where it stands, overlap and boundaries included."""
    os.environ["LLOGOS_RUNNER"] = "0"           # the parts call the kernels one by one, so each can be left out
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = L.weights.random_model(cfg, seed=0, dtype=torch.bfloat16, device=dev, std=0.02)
    gen = torch.Generator().manual_seed(1)
    names = ("add_rmsnorm", "qk_prep", "attn_decode", "gemm_tc")
    real = {n: getattr(ops, n) for n in names}
    q_rows = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    h, inter, vocab, n_layers = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]

    def measure(patch):
        for n, f in real.items():
            setattr(ops, n, f)
        patch()
        eng = L.engine.Engine(model, max_tokens=batch * pages_of(context), max_seq_len=context, n_slots=batch)
        steps, warmup = 16, 4
        slots = [eng.open() for _ in range(batch)]
        for s in slots:
            eng.assume(s, context - (steps + warmup))
        tok = torch.randint(0, vocab, (steps + warmup, batch), generator=gen).tolist()
        for i in range(warmup):
            eng.step([(s, [tok[i][j]]) for j, s in enumerate(slots)])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            eng.step([(s, [tok[i][j]]) for j, s in enumerate(slots)])
        e1.record()
        torch.cuda.synchronize()
        del eng
        torch.cuda.empty_cache()
        return e0.elapsed_time(e1) / steps

    def without_product(pred):
        def f(x, w, out, **kw):
            if not pred(w, kw):
                real["gemm_tc"](x, w, out, **kw)
        return lambda: setattr(ops, "gemm_tc", f)

    base = measure(lambda: None)
    print(f"batch {batch} context {context}: whole step {base:.3f} ms, {base / n_layers * 1e3:.1f} us per layer (head included)")
    cases = [("add_rmsnorm (two per layer)", lambda: setattr(ops, "add_rmsnorm", lambda *a, **k: None), n_layers),
             ("qk_prep", lambda: setattr(ops, "qk_prep", lambda *a, **k: None), n_layers),
             ("attn_decode", lambda: setattr(ops, "attn_decode", lambda *a, **k: None), n_layers),
             ("q/k/v product", without_product(lambda w, kw: w.shape[0] == q_rows and not kw.get("gated_features")), n_layers),
             ("output product", without_product(lambda w, kw: tuple(w.shape) == (h, cfg["num_attention_heads"] * cfg["head_dim"])
                                                and w.shape[0] != q_rows), n_layers),
             ("gate/up product", without_product(lambda w, kw: kw.get("gated_features", 0) > 0), n_layers),
             ("down product", without_product(lambda w, kw: tuple(w.shape) == (h, inter)), n_layers),
             ("head product", without_product(lambda w, kw: w.shape[0] == vocab), 1)]
    for label, patch, per in cases:
        ms = measure(patch)
        print(f"  without {label:30s} {ms:.3f} ms: {(base - ms) * 1e3 / per:7.1f} us each", flush=True)
    return 0


def probe_timeline(torch, L, ops, cfg, batch, context, prompt_tokens=0):
    """One decode step's kernels (or, with `prompt_tokens`, those of one prompt step of so many tokens) on one time line, from stamps that the kernels themselves leave (%globaltimer, 32 ns
    steps) when the library is built with LLOGOS_NVCC_FLAGS=-DLLG_STAMPS: for every launch its number of blocks, when
    its first and last block started, when their dependency wait returned, when the products were done and when the
    blocks ended, in microseconds from the step's first stamp.  A stamp costs about a third of a microsecond."""
    import ctypes
    import numpy as np
    if "-DLLG_STAMPS" not in os.environ.get("LLOGOS_NVCC_FLAGS", "").split():
        print("the time line needs the kernels built with their stamps: run with LLOGOS_NVCC_FLAGS=-DLLG_STAMPS")
        return 2
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = L.weights.random_model(cfg, seed=0, dtype=torch.bfloat16, device=dev, std=0.02)
    eng = L.engine.Engine(model, max_tokens=batch * pages_of(context), max_seq_len=context, n_slots=batch)
    for g in eng.cache.kv_groups:
        for t in list(g.k.values()) + list(g.v.values()):
            t.normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(1)
    if prompt_tokens > 0:
        prompt = torch.randint(0, cfg["vocab_size"], (prompt_tokens,), generator=gen).tolist()

        def step(i):
            slot = eng.open()
            eng.step([(slot, prompt)])
            eng.close(slot)
    else:
        slots = [eng.open() for _ in range(batch)]
        for s in slots:
            eng.assume(s, context - 40)
        tok = torch.randint(0, cfg["vocab_size"], (13, batch), generator=gen).tolist()

        def step(i):
            eng.step([(s, [tok[i][j]]) for j, s in enumerate(slots)])
    libs = [ops._lib(n) for n in ("gemm_tc", "attention_decode_tma", "attention_tc", "elementwise")]
    cap = 131072

    def read():
        parts = []
        for lib in libs:
            buf = (ctypes.c_ulonglong * (2 * cap))()
            lib.llg_stamps_read.argtypes = [ctypes.c_void_p, ctypes.c_int]
            lib.llg_stamps_read.restype = ctypes.c_int
            k = lib.llg_stamps_read(buf, cap)
            parts.append(np.frombuffer(buf, dtype=np.uint64)[: 2 * k].reshape(-1, 2).copy())
        return np.concatenate(parts)

    for i in range(12):
        step(i)
    read()                                       # the warm-up steps' stamps are dropped
    step(12)
    st = read()
    t, tag = st[:, 0].astype(np.int64), st[:, 1]
    kern = (tag >> np.uint64(56)).astype(int)
    phase = ((tag >> np.uint64(48)) & np.uint64(0xff)).astype(int)
    aux = ((tag >> np.uint64(32)) & np.uint64(0xffff)).astype(int)
    aux[kern != 1] = 0
    t = (t - t.min()) / 1000.0
    h, inter = cfg["hidden_size"], cfg["intermediate_size"]
    q_rows = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    tag_of = lambda k, rows: (((k >> 10) & 0xff) << 8) | ((rows >> 9) & 0xff)
    names = {tag_of(h, q_rows): "q/k/v", tag_of(cfg["num_attention_heads"] * cfg["head_dim"], h): "output",
             tag_of(h, 2 * inter): "gate/up", tag_of(inter, h): "down", tag_of(h, cfg["vocab_size"]): "head"}
    other = {2: "attention", 3: "norm", 4: "qk_prep", 5: "attention"}
    rows = []
    for key in sorted(set(zip(kern.tolist(), aux.tolist()))):
        m = (kern == key[0]) & (aux == key[1])
        tt, ph = t[m], phase[m]
        order = np.argsort(tt, kind="stable")
        tt, ph = tt[order], ph[order]
        starts = tt[ph == 0]
        # a kernel's launches: a block that starts well after the one before, with a block's end in between, belongs
        # to the next launch (or to the next wave of a grid larger than the device holds: the head product's)
        ends = tt[ph == 3]
        cuts = [0] + [i + 1 for i in range(len(starts) - 1) if starts[i + 1] - starts[i] > 15.0
                      and ((ends > starts[i]) & (ends < starts[i + 1])).any()] + [len(starts)]
        for a, b in zip(cuts[:-1], cuts[1:]):
            nxt = starts[b] if b < len(starts) else float("inf")
            sel = (tt >= starts[a]) & (tt < nxt)
            span = lambda q: ((tt[sel & (ph == q)].min(), tt[sel & (ph == q)].max()) if (sel & (ph == q)).any()
                              else (float("nan"), float("nan")))
            name = names.get(key[1], f"product {key[1]:#x}") if key[0] == 1 else other.get(key[0], str(key[0]))
            rows.append((starts[a], name, b - a, (starts[a], starts[b - 1]), span(1), span(2), span(3)))
    rows.sort(key=lambda r: r[0])
    what = f"prompt of {prompt_tokens} tokens" if prompt_tokens > 0 else f"batch {batch} context {context}"
    print(f"{what}, {cfg['num_hidden_layers']} layers: {len(t)} stamps; microseconds from the first")
    print(f"{'kernel':10s} {'blocks':>6s} {'start':>15s} {'wait returned':>15s} {'products done':>15s} {'end':>15s}")
    for r in rows:
        print(f"{r[1]:10s} {r[2]:6d} " + " ".join(f"{a:7.1f}-{b:7.1f}" for a, b in r[3:]))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="llama-3.1-8b", choices=sorted(SHAPES), help="layer sizes (default: the headline shape)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length of the decode steps (default 8192)")
    ap.add_argument("--layers", type=int, default=0,
                    help="layers to build (default: all of the shape's); both numbers are reported")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="leave out the workloads of the other shapes and the ragged run")
    ap.add_argument("--tokens", type=int, default=0,
                    help="with --probe timeline: the time line of a prompt step of so many tokens instead of a decode step")
    ap.add_argument("--probe", choices=["decode-attention", "leave-one-out", "timeline"],
                    help="instead of the bench line, print a table: decode attention alone over batch shapes; what "
                         "the decode step loses when each kernel in turn is left out of the recorded graph; or one "
                         "decode step's launches on a time line (needs LLOGOS_NVCC_FLAGS=-DLLG_STAMPS; --layers, default 6)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a .NET 10 / C# solution (no Python package, no dotnet SDK in this image): "
                          "pip cannot install it and its CLI cannot be built here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import importlib
    import torch
    L = importlib.import_module("llogos_b200")
    ops = importlib.import_module("daisi-llogos_b200.kernels.ops")
    pk = peaks()
    if args.probe == "decode-attention":
        return probe_decode_attention(torch, ops, SHAPES[args.shape][1], pk)
    if args.probe == "leave-one-out":
        return probe_leave_one_out(torch, L, ops, dict(SHAPES[args.shape][1]), args.batch, args.context)
    if args.probe == "timeline":
        return probe_timeline(torch, L, ops, dict(SHAPES[args.shape][1], num_hidden_layers=args.layers or 6),
                              args.batch, args.context, args.tokens)
    shape_name, shape = SHAPES[args.shape]
    if args.layers <= 0:
        args.layers = shape["num_hidden_layers"]
    context = args.context
    cfg = dict(shape, num_hidden_layers=args.layers)
    nums = model_numbers(cfg, args.layers)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)

    t0 = time.time()
    model = L.weights.random_model(cfg, seed=0, dtype=torch.bfloat16, device=dev, std=0.02)
    big = args.batch if args.no_points else max(64, args.batch)
    weight_gb = (nums["matrix_params"] + 2 * nums["head_params"]) * 2 / 1e9
    if weight_gb + big * context * nums["kv_bytes_per_token"] / 1e9 > 165.0:
        # the cache of 64 sequences at this context does not fit beside the weights: no batch-64 point
        big = args.batch
    engine = L.engine.Engine(model, max_tokens=big * pages_of(context), max_seq_len=context, n_slots=big)
    for g in engine.cache.kv_groups:             # random keys and values: attention over real numbers
        for t in list(g.k.values()) + list(g.v.values()):
            t.normal_(0.0, 1.0)
    torch.cuda.synchronize()
    print(f"[bench] model and cache ready in {time.time() - t0:.1f} s "
          f"(weights {(nums['matrix_params'] + 2 * nums['head_params']) * 2 / 1e9:.2f} GB, cache {engine.cache.bytes() / 1e9:.1f} GB)",
          file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(1)

    # ---- prefill of 2,048 tokens ------------------------------------------------------------
    toks = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for it in range(3 + 5):
        slot = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([(slot, toks)])
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
        engine.close(slot)
    pre_ms = sorted(times)[len(times) // 2]
    # prompt steps back to back run into the power cap; one more after half a second of idle shows the
    # step as a lone request meets it (reported beside the back-to-back median, which stays the headline)
    time.sleep(0.5)
    slot = engine.open()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    engine.step([(slot, toks)])
    e1.record()
    torch.cuda.synchronize()
    idle_ms = e0.elapsed_time(e1)
    engine.close(slot)
    t = PREFILL_TOKENS
    attn_flops = args.layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * (t * (t + 1) / 2)
    pre_flops = 2.0 * t * nums["matrix_params"] + 2.0 * nums["head_params"] + attn_flops
    prefill = {"value": round(t / (pre_ms / 1e3), 1), "tokens": t, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "ms_after_idle": round(idle_ms, 3)}
    if pk.get("bf16_tflops_sustained"):       # back-to-back steps run under the power cap: the sustained figure is their peak
        prefill["frac_sustained"] = round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)

    # ---- decode steps at the context length --------------------------------------------------
    def decode(batch, steps, warmup, clocks=None):
        slots = [engine.open() for _ in range(batch)]
        start = context - (steps + warmup)
        for s in slots:
            engine.assume(s, start)
        tok = torch.randint(0, cfg["vocab_size"], (steps + warmup, batch), generator=gen).tolist()
        for i in range(warmup):
            engine.step([(s, [tok[i][j]]) for j, s in enumerate(slots)])
        torch.cuda.synchronize()
        k0, l0 = engine.graph_kernels, ops.launches()
        if clocks:
            clocks.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            engine.step([(s, [tok[i][j]]) for j, s in enumerate(slots)])
        e1.record()
        torch.cuda.synchronize()
        if clocks:
            clocks.stop()
        ms = e0.elapsed_time(e1) / steps
        launches = (engine.graph_kernels - k0) + (ops.launches() - l0)
        mean_len = start + warmup + (steps + 1) / 2.0
        for s in slots:
            engine.close(s)
        return ms, launches, mean_len

    clocks = Clocks()
    ms, launches, mean_len = decode(args.batch, args.steps, args.warmup, clocks)
    value = args.batch / (ms / 1e3)
    weight_bytes = (nums["matrix_params"] + nums["head_params"]) * 2 + args.batch * cfg["hidden_size"] * 2
    step_bytes = weight_bytes + args.batch * mean_len * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]}
    print(f"[bench] decode b{args.batch}: {ms:.3f} ms/step, {value:.1f} tok/s, {roofline}", file=sys.stderr, flush=True)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            if b > big:
                points[f"decode_b{b}"] = None
                continue
            pms, _, _ = decode(b, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 1)
            print(f"[bench] decode b{b}: {pms:.3f} ms/step", file=sys.stderr, flush=True)

    # ---- the same batch through the Python entry point ----------------------------------------
    e2e = None
    del engine
    torch.cuda.empty_cache()
    api = None
    if not args.no_e2e:
        api = L.LlogosModel(model, max_context=context, max_batch=args.batch)
        # A request's own prompt (8 x 8k tokens, most of a second at the power cap) leaves the SM clock
        # throttled for the first twenty or so decode steps; they are run untimed, as warm-up steps are,
        # and the K steps after them are timed on the host from the moments their tokens arrive.
        untimed = max(args.warmup, 32)
        n_new = untimed + args.steps
        prompts = [torch.randint(0, cfg["vocab_size"], (context - n_new - 1,), generator=gen).tolist() for _ in range(args.batch)]
        params = L.GenerationParams.greedy_params(n_new, stop_tokens=())
        api.generate([p[:64] for p in prompts], L.GenerationParams.greedy_params(args.warmup + 2, stop_tokens=()))   # warm-up: graph capture
        stamps = []

        def on_token(request, token):
            if request == args.batch - 1:
                stamps.append(time.perf_counter())

        r = api.generate(prompts, params, on_token=on_token)
        assert len(stamps) == n_new and r.generated_tokens == n_new * args.batch
        e2e_s = stamps[-1] - stamps[untimed - 1]
        e2e = {"value": round(args.steps * args.batch / e2e_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": (7 * args.batch + 1) * 4, "d2h_bytes_per_step": args.batch * 4,
               "ms_per_step": round(e2e_s / args.steps * 1e3, 4), "untimed_steps": untimed,
               "whole_call_tokens_per_s": round(r.decode_tokens_per_second, 1),
               "prefill_tokens_per_s": round(r.prefill_tokens_per_second, 1), "decode_steps": r.decode_steps}
        print(f"[bench] e2e {e2e}", file=sys.stderr, flush=True)

    # ---- the workloads as they are written ------------------------------------------------------
    if not args.no_workloads and not args.no_points and args.shape == "llama-3.1-8b" and args.layers == shape["num_hidden_layers"]:
        measure = importlib.import_module("daisi-llogos_b200.measure")
        import random

        def workload(api, tag, lo, hi, batch, *, steps=None, to_context=None, temperature=0.0):
            rng = random.Random(7)
            vocab = api.model.spec.vocab_size
            prompts = [[rng.randrange(vocab) for _ in range(rng.randint(lo, hi))] for _ in range(batch)]
            n_new = steps if steps is not None else to_context
            if temperature == 0.0:
                params = L.GenerationParams.greedy_params(n_new, stop_tokens=())
            else:
                params = L.GenerationParams(max_tokens=n_new, temperature=temperature, top_k=0, top_p=1.0,
                                            repetition_penalty=1.0, seed=1, stop_tokens=())
            api.generate([p[:64] for p in prompts], L.GenerationParams.greedy_params(4, stop_tokens=()))       # graphs
            if steps is not None:
                # A run of a few hundred steps: the first call records the decode steps' graphs for its batch size and
                # length bounds (and loads kernels that no earlier call used), which takes a tenth to a third of such a
                # run's decode time and varies; the call that is timed is the second, as a server that is up would see it.
                api.generate(prompts, params)
            r = api.generate(prompts, params)
            costs = measure.model_costs(api.model)
            lens, made = [len(p) for p in prompts], [len(t) for t in r.tokens]
            nbytes, n_steps = measure.decode_bytes_of_run(costs, lens, made)
            frac = nbytes / r.decode_seconds / 1e9 / pk["hbm_gbs"] if r.decode_seconds > 0 else None
            points[tag] = round(r.decode_tokens_per_second, 1)
            points[tag + "_hbm_frac"] = round(frac, 4) if frac else None
            points[tag + "_prefill_tok_s"] = round(r.prefill_tokens_per_second, 1)
            print(f"[bench] {tag}: {points[tag]} tok/s over {r.decode_steps} decode steps, {points[tag + '_hbm_frac']} of the copy "
                  f"bandwidth; prompts {r.prompt_tokens} tokens at {points[tag + '_prefill_tok_s']} tok/s; longest sequence at the "
                  f"end {max(a + b for a, b in zip(lens, made))}", file=sys.stderr, flush=True)

        try:
            if api is None:
                api = L.LlogosModel(model, max_context=context, max_batch=args.batch)
            workload(api, "llama8b_b8_ragged_to_8192", 128, 2048, args.batch, to_context=context)
        except Exception as e:                                   # a point that cannot run is reported, not fatal
            points["llama8b_b8_ragged_to_8192"] = None
            print(f"[bench] llama8b_b8_ragged_to_8192 failed: {e}", file=sys.stderr, flush=True)
        del api, model
        torch.cuda.empty_cache()
        for tag, cfg2, batch, lo, hi, steps, temps in (
                ("qwen3_8b_b16_256steps", QWEN3_8B, 16, 64, 4096, 256, (0.0, 0.7)),
                ("qwen25_14b_b32_128steps", QWEN25_14B, 32, 256, 8192, 128, (0.0,))):
            try:
                api2 = L.LlogosModel.random(cfg2, seed=0, dtype="bfloat16", max_context=hi + steps, max_batch=batch, std=0.02)
                for t in temps:
                    name = tag if len(temps) == 1 else f"{tag}_{'greedy' if t == 0.0 else 't' + str(t)}"
                    workload(api2, name, lo, hi, batch, steps=steps, temperature=t)
                del api2
            except Exception as e:
                points[tag] = None
                print(f"[bench] {tag} failed: {e}", file=sys.stderr, flush=True)
            torch.cuda.empty_cache()
        # the 32-bit path against the bfloat16 path on one short sequence, two layers of the 14B shape's 48
        try:
            small = dict(QWEN25_14B, num_hidden_layers=2)
            toks2 = torch.randint(0, small["vocab_size"], (96,), generator=gen).tolist()
            got = {}
            for dt in (torch.float32, torch.bfloat16):
                m2 = L.weights.random_model(small, seed=0, dtype=dt, device=dev, std=0.02)
                e2 = L.engine.Engine(m2, max_tokens=128)
                got[dt] = e2.step([(e2.open(), toks2)], [list(range(96))]).double().cpu()
                del e2, m2
                torch.cuda.empty_cache()
            rel = float((got[torch.float32] - got[torch.bfloat16]).abs().max() / got[torch.float32].abs().max())
            points["qwen25_14b_2of48_layers_fp32_vs_bf16_max_rel_diff"] = round(rel, 5)
            print(f"[bench] 32-bit path against bfloat16, 96 tokens, 2 of 48 layers of the 14B shape: {rel:.5f} of the largest logit",
                  file=sys.stderr, flush=True)
        except Exception as e:
            print(f"[bench] 32-bit cross-check failed: {e}", file=sys.stderr, flush=True)

    line = {
        "metric": f"decode tokens/s at batch {args.batch}, context {context} ({shape_name}, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform random token ids, random cache contents",
        "impl": "ours",
        "config": {"model": shape_name, "layers": args.layers, "layers_of_config": shape["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "rope_theta": cfg["rope_theta"],
                   "rope_scaling": "llama3 factor 8 low 1 high 4 original 8192" if cfg.get("rope_scaling") else "none",
                   "global_batch": args.batch, "seq_len": context, "parallelism": "single GPU",
                   "l2": "every step reads more than L2 holds (weights + cache), no flush",
                   "cache": "pages of 64 tokens, bf16", "decode": "CUDA graph per batch size"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": int(launches), "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
