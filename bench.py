"""Decode and prefill throughput of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests whose contexts end at 4,096 tokens. `value` is
decoded tokens per second timed on the device with CUDA events around exactly K steps (each step:
the batch tables copied to the device, the captured decode graph replayed, argmax on the device);
`e2e` is the same through the public entry point (`Engine.add_request` / `Engine.step_once`): host
token lists in, sampled tokens read back on the host every step (the engine plans and launches a step
while the one before runs, so the tokens it reads are those of the step before), prompts prefilled by
the engine itself. `prefill` times one 2,048-token prompt; `roofline` compares the bytes a decode step has to
read (every weight once plus the cache of the live requests) with the measured copy bandwidth;
`points` holds decode at batch 1 and 64; `check` compares the bfloat16 logits with the 32-bit path's at these
layer sizes (two layers, untimed). Peaks come from MEASURED_PEAKS.json when it exists.

`--design madevik`, `--design movivik`, `--design bozevik` and `--design guvolix` are another program under the same roof and leave the default
workload alone: prefill and decode of the Madevik design (gated linear attention, attention over a cached latent, routed
experts), of the Movivik design (chunked and parallel attention layers, linear attention with fixed decays, norms in front of
and behind every part) or of the Bozevik design (attention over a cached latent with a query latent and a shared rotated key
part, layer norms behind the parts, token shift, depth mix, clamped gated units) or of the Guvolix design (one norm per
layer that feeds an attention with a sink and kept first tokens beside a selective state space or a matrix memory, and a
dense or routed feed-forward) at layer sizes that resemble a real model's, beside the Qwen3 dense shape of the same width, heads, layers and feed-forward weights (`--design-sizes`
picks among them); one JSON line with both models' figures per size.

The engine runs on one GPU; for --gpus above 1 the program says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                attention_bias=False, use_sliding_window=False, max_position_embeddings=40960, hidden_act="silu")
# the layer shapes of BASELINE.json's other configurations (same architecture; random weights): --shape
SHAPES = {"8b": QWEN3_8B,
          "14b": dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, intermediate_size=17408),
          "32b": dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, intermediate_size=25600)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in raw:
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg: dict, layers: int) -> dict:
    D, H, Hkv, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                           cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = D * (H + 2 * Hkv) * hd + H * hd * D + 3 * D * F
    return {"layer_params": per_layer, "head_params": V * D, "weight_bytes": 2 * (per_layer * layers + V * D),
            "kv_bytes_per_token": 2 * layers * Hkv * hd * 2,
            "attn_flops_per_layer": lambda T: 4 * (T * (T + 1) // 2) * H * hd}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": 1.5}}


def madevik_shape(width, heads, rank, experts, top, ff, runs, vocab=32768):
    """Every fourth layer, from the second on, attends over a cached latent, the others are linear attention; head size 128
    throughout."""
    mlp = _moe(experts, top, ff)
    gla = {"type": "gla", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "tau": 8.0, "decay_rank": 64}, "mlp": mlp}
    latent = {"type": "latent_attention",
              "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": rank, "scale": 128 ** -0.5}, "mlp": mlp}
    return {"architecture": "Madevik", "width": width, "vocab": vocab, "residual_mult": 0.7, "norm": {"eps": 1e-6},
            "layers": [latent if i % 4 == 1 else gla for i in range(runs)]}


def movivik_shape(width, heads, kv_heads, ff, runs, chunk=1024, vocab=32768):
    """Layers in pairs: two of chunked attention (YaRN-scaled interleaved rotation, biases), then two parallel layers (a
    causal attention that rotates half of every head and norms q and k, beside linear attention with a fixed decay per
    head); head size 128 throughout, a dense GELU-gated feed-forward in every layer."""
    mlp = {"kind": "dense", "ff": ff}
    att = {"type": "attention", "mlp": mlp, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": chunk},
        "rot": {"base": 500000.0, "dims": 128, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}}
    decay = [1.0 - 2.0 ** (-2 - 6 * h / max(1, heads - 1)) for h in range(heads)]
    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "rot": {"base": 10000.0, "dims": 64}},
        "right": {"heads": heads, "dim": 128, "vdim": 128, "decay": decay}}}
    return {"architecture": "Movivik", "width": width, "vocab": vocab, "norm": {"eps": 1e-6},
            "layers": [att if i % 4 < 2 else par for i in range(runs)]}


def bozevik_shape(width, heads, rank, rot, q_rank, experts, top, ff, dense_ff, runs, vocab=32768):
    """Attention over a cached latent in every layer (queries through a latent of `q_rank` values, a rotated key part of `rot`
    values beside a latent of `rank`; every second layer reads the rows the layer in front of it cached), head size 128; dense
    and routed feed-forwards (with a shared expert) take turns."""
    def mixer(i):
        m = {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": rank, "q_rank": q_rank, "rot_dim": rot,
             "rot": {"base": 10000.0, "dims": rot}, "scale": (128 + rot) ** -0.5}
        return dict(m, kv_from=i - 1) if i % 2 else m
    dense = {"kind": "dense", "ff": dense_ff, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top},
           "shared": {"ff": ff, "limit": 7.0}}
    return {"architecture": "Bozevik", "width": width, "vocab": vocab, "logit_scale": 1.0, "norm": {"eps": 1e-6},
            "layers": [{"type": "latent_attention", "mixer": mixer(i), "mlp": moe if i % 2 else dense} for i in range(runs)]}


def madevik_latent_shape(width, heads, rank, experts, top, ff, runs, vocab=32768):
    """A Madevik model of latent-attention layers only (the closest kin of the Bozevik shape): cached rows of `rank` values."""
    latent = {"type": "latent_attention", "mlp": _moe(experts, top, ff),
              "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": rank, "scale": 128 ** -0.5}}
    return {"architecture": "Madevik", "width": width, "vocab": vocab, "residual_mult": 0.7, "norm": {"eps": 1e-6},
            "layers": [latent for _ in range(runs)]}


def guvolix_shape(width, heads, kv_heads, ff, runs, window=1024, keep=64, vocab=32768):
    """Layers in fours: three whose attention (a window with kept first tokens, a sink, a gate of full width) runs beside a
    selective state space (inner width twice the model's, heads of 64 values, states of 128, eight groups), one whose attention
    (a window, banded rotary scaling) runs beside a matrix memory (heads of 128 key and 256 value channels); attention heads of
    128 throughout; a dense erf-GELU feed-forward and routed experts (softmax scores, two identity entries, a gated shared
    expert) take turns."""
    def left(p2):
        rot = {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0}}
        mask = {"size": window, "keep_first": keep}
        if p2:
            rot = {"base": 20000.0, "dims": 128, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 4096}}
            mask = {"size": window}
        return {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": rot, "mask": mask}
    ssm = {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}
    mem = {"heads": width // 256, "dim": 128, "vdim": 256, "gate_cap": 15.0}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // 8}, "router": {"experts": 8, "top": 2, "identity": 2}, "shared": {"ff": ff // 8}}
    layers = []
    for i in range(runs):
        mlp = moe if i % 2 else dense
        if i % 4 == 3:
            layers.append({"type": "parallel_2", "mlp": mlp,
                           "mixer": {"left": left(True), "right": mem, "left_scale": 0.6, "right_scale": 1.1}})
        else:
            layers.append({"type": "parallel", "mlp": mlp, "mixer": {"left": left(False), "right": ssm}})
    return {"architecture": "Guvolix", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
            "layers": layers}


def movivik_parallel_shape(width, heads, kv_heads, ff, runs, vocab=32768):
    """A Movivik model of parallel layers only (the closest kin of the Guvolix shape): a causal attention beside linear
    attention with a fixed decay per head, heads of 128, a dense gated feed-forward."""
    cfg = movivik_shape(width, heads, kv_heads, ff, runs, vocab=vocab)
    par = [l for l in cfg["layers"] if l["type"] == "parallel"][0]
    return dict(cfg, layers=[par for _ in range(runs)])


def _qwen3_shape(width, layers, heads, kv_heads, ffn):
    return dict(QWEN3_8B, hidden_size=width, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
                intermediate_size=ffn, vocab_size=32768)


# design -> name -> (the design's configuration, the Qwen3 dense shape of the same width, heads, layers and feed-forward
# weights[, a third configuration and its label: the design's closest kin among the other designs])
DESIGN_SIZES = {
    "madevik": {"w2048": (madevik_shape(2048, 16, 128, 8, 2, 1024, 8), _qwen3_shape(2048, 8, 16, 8, 8192)),
                "w4096": (madevik_shape(4096, 32, 256, 16, 4, 768, 4), _qwen3_shape(4096, 4, 32, 8, 12288))},
    "movivik": {"w2048": (movivik_shape(2048, 16, 8, 8192, 8), _qwen3_shape(2048, 8, 16, 8, 8192)),
                "w4096": (movivik_shape(4096, 32, 8, 12288, 4), _qwen3_shape(4096, 4, 32, 8, 12288))},
    # cached rows of 192 + 64 and of 96 + 32 values; beside each the Qwen3 shape and a Madevik model of latent-attention
    # layers with cached rows of the same width and the same experts
    "bozevik": {"w2048": (bozevik_shape(2048, 16, 192, 64, 768, 8, 2, 1024, 8192, 8), _qwen3_shape(2048, 8, 16, 8, 8192),
                          madevik_latent_shape(2048, 16, 256, 8, 2, 1024, 8), "madevik_latent"),
                "w4096": (bozevik_shape(4096, 32, 96, 32, 1536, 16, 4, 768, 12288, 4), _qwen3_shape(4096, 4, 32, 8, 12288),
                          madevik_latent_shape(4096, 32, 128, 16, 4, 768, 4), "madevik_latent")},
    # beside each the Qwen3 shape and a Movivik model of parallel layers (attention beside linear attention)
    "guvolix": {"w2048": (guvolix_shape(2048, 16, 8, 8192, 8), _qwen3_shape(2048, 8, 16, 8, 8192),
                          movivik_parallel_shape(2048, 16, 8, 8192, 8), "movivik_parallel"),
                "w4096": (guvolix_shape(4096, 32, 8, 12288, 4), _qwen3_shape(4096, 4, 32, 8, 12288),
                          movivik_parallel_shape(4096, 32, 8, 12288, 4), "movivik_parallel")},
}


def design_bench(args) -> int:
    """Prefill of one prompt and decode steps of a batch, device-timed, for the chosen design and the Qwen3 dense shape
    beside it. Decode: `--batch` requests whose contexts (synthetic cache content, zero states) stand at `--context`."""
    import torch

    from jllm_serve_b200.csrc import ops
    from jllm_serve_b200.engine import Engine, Segment

    ctx, batch, tokens = min(args.context, 2048), args.batch, min(PREFILL_TOKENS, args.context)
    steps, warmup = max(8, args.steps // 2), max(3, args.warmup)
    sizes = DESIGN_SIZES[args.design]
    out = {"design": args.design, "dtype": "bf16", "data": "synthetic token ids, random-init weights", "prefill_tokens": tokens,
           "decode_batch": batch, "decode_context": ctx, "steps": steps, "warmup": warmup, "sizes": {}}
    out_tok = torch.empty(max(64, batch), dtype=torch.int32, device="cuda:0")
    for name in args.design_sizes.split(","):
        if name not in sizes:
            print(f"bench.py: unknown size {name!r} (known: {', '.join(sorted(sizes))})")
            return 2
        record = {}
        entry = sizes[name]
        for model, cfg in zip((args.design, "qwen3") + tuple(entry[3:4]), entry[:3]):
            engine = Engine(config=cfg, seed=0, dtype="bfloat16", ctx=ctx + 64, page_size=PAGE,
                            num_pages=((batch + 1) * (ctx + 64) + 2 * tokens) // PAGE, max_batch_tokens=tokens + 64,
                            chunk=tokens, max_running=batch + 2)
            runner = engine.runner
            print(f"bench: {runner.describe()}", file=sys.stderr, flush=True)
            for g in runner.cache.paged:
                g.storage.normal_()
            gen = torch.Generator().manual_seed(1)
            prompt = torch.randint(0, runner.vocab, (tokens,), generator=gen).tolist()
            times = []
            for i in range(7):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                runner.step([Segment(f"p{i}", prompt, 0, [tokens - 1])])
                e.record()
                torch.cuda.synchronize()
                runner.finish(f"p{i}")
                times.append(s.elapsed_time(e))
            pre_ms = statistics.median(times[2:])
            ids = [f"d{i}" for i in range(batch)]
            start = ctx - warmup - steps
            for i in ids:
                runner.cache.open(i)
                runner.cache.reserve(i, 0, start)
                runner.cache.commit(i, start)

            def one_step():
                logits = runner.step([Segment(i, [1 + k], runner.cache.length(i), [0]) for k, i in enumerate(ids)])
                ops.argmax(logits, out_tok[:batch])

            for _ in range(warmup):
                one_step()
            torch.cuda.synchronize()
            before = ops.launch_count
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(steps):
                one_step()
            e.record()
            torch.cuda.synchronize()
            dec_ms = s.elapsed_time(e) / steps
            launches = (ops.launch_count - before) // steps
            for i in ids:
                runner.finish(i)
            weights = sum(t.numel() * t.element_size() for t in _tensors_of(runner.model))
            record[model] = {"prefill_ms": round(pre_ms, 3), "prefill_tokens_per_s": round(tokens / pre_ms * 1e3, 1),
                             "decode_ms_per_step": round(dec_ms, 4), "decode_tokens_per_s": round(batch * 1e3 / dec_ms, 1),
                             "kernels_per_decode_step": launches, "weight_gb": round(weights / 1e9, 3),
                             "layers": len(runner.spec.schedule)}
            engine.close()
            del engine, runner
            torch.cuda.empty_cache()
        out["sizes"][name] = record
    print(json.dumps(out))
    return 0


def _tensors_of(obj, seen=None):
    """Every device tensor reachable from a model's parts (weights, packed or plain), each once."""
    import torch
    seen = set() if seen is None else seen
    if id(obj) in seen:
        return
    seen.add(id(obj))
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda and obj.data_ptr() not in seen:
            seen.add(obj.data_ptr())
            yield obj
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _tensors_of(v, seen)
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _tensors_of(v, seen)
    elif hasattr(obj, "__dict__") and type(obj).__module__.startswith("jllm_serve_b200") and type(obj).__name__ != "Runtime":
        for v in vars(obj).values():
            yield from _tensors_of(v, seen)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--design", default="", choices=["", "madevik", "movivik", "bozevik", "guvolix"],
                    help="madevik, movivik, bozevik, guvolix: time that design beside the Qwen3 dense shape of equal size (bozevik: "
                         "also beside a Madevik model of latent-attention layers; guvolix: also beside a Movivik model of "
                         "parallel layers) instead of the default workload")
    ap.add_argument("--design-sizes", default="w2048,w4096", help="which of the sizes of --design, with commas between them")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--rounds", type=int, default=5,
                    help="the K steps are timed this many times, one after the other; the median round is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (named in the record)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: Qwen3-8B (default), 14B or 32B")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length at which the decode steps are timed")
    ap.add_argument("--mixed-chunk", type=int, default=0,
                    help="rows of a prompt portion that rides in every timed step beside the decoding requests")
    ap.add_argument("--kv-share", type=float, default=0.0,
                    help="size the cache pool as this share of the device memory left after the weights (else: the "
                         "pages the run needs)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--prefill-only", action="store_true", help="profiling aid: time the prefill alone and print it")
    ap.add_argument("--skip-check", action="store_true",
                    help="leave out the comparison of the bfloat16 path with the 32-bit path at these layer sizes")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "beniaminp/jllm-serve is a Java 26 program with an Apple "
                          "Metal GPU path (no Python package, no CUDA code): pip cannot install it and no JDK is present"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    args.warmup = max(3, args.warmup)
    if args.design:
        return design_bench(args)

    import torch

    from jllm_serve_b200.csrc import ops
    from jllm_serve_b200.engine import Engine, Segment
    from jllm_serve_b200.sampling import SamplingParams

    shape = SHAPES[args.shape]
    args.layers = args.layers or shape["num_hidden_layers"]
    ctx = args.context
    default_run = args.shape == "8b" and ctx == CONTEXT and not args.mixed_chunk
    if not default_run:
        args.skip_points = args.skip_e2e = True
    cfg = dict(shape, num_hidden_layers=args.layers)
    nums = model_numbers(cfg, args.layers)
    pk = peaks()
    dev = torch.device("cuda:0")
    biggest = 64 if not args.skip_points else args.batch
    pool_tokens = biggest * ctx + 2 * PREFILL_TOKENS + args.mixed_chunk
    check = None
    if not (args.skip_check or args.prefill_only):
        # the 32-bit path against the bfloat16 path at these layer sizes, on two layers (untimed, before the model)
        from jllm_serve_b200.precision_check import compare_precisions
        # (a prompt of 1,280 rows in portions of 1,024, so that the products of many rows are the ones the prefill takes)
        got = compare_precisions(dict(shape, num_hidden_layers=2), seed=0, prompt=1280, tail=16, portion=1024)["mixed"]
        check = {"what": "bfloat16 logits against the 32-bit path, a 1024+256-row prompt beside 2 decoding requests, "
                         "then 16 tokens one by one", "layers": 2, "layers_of_config": shape["num_hidden_layers"],
                 "rows": got["rows"], "max_rel": round(got["max_rel"], 5), "rms_rel": round(got["rms_rel"], 5),
                 "argmax_agree": round(got["argmax_agree"], 4), "choice_gap_rel": round(got["worst_choice_gap_rel"], 5)}
    t0 = time.time()
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", ctx=ctx, page_size=PAGE,
                    num_pages="auto" if args.kv_share > 0 else pool_tokens // PAGE, kv_share=args.kv_share or 0.6,
                    max_batch_tokens=PREFILL_TOKENS + 64, chunk=PREFILL_TOKENS, max_running=biggest + 1)
    runner = engine.runner
    print(f"bench: {runner.describe()} (built in {time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    for note in runner.notes:
        print(f"bench: {note}", file=sys.stderr, flush=True)
    for g in runner.cache.paged:      # any cached values do for timing; zeros would be kinder to the memory system
        g.storage.normal_()
    out_tok = torch.empty(64, dtype=torch.int32, device=dev)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def decode_device_timed(batch: int, steps: int, warmup: int, rounds: int = 1):
        """`batch` requests whose contexts END at the context length after warmup + rounds x steps decoded tokens;
        the cache content is synthetic. With --mixed-chunk a portion of a prompt (rows 1,024 onwards of a request
        that is given back after the step) runs in every step before them. Each round times exactly `steps` steps
        between two events with a synchronize on both sides; the median round is reported.
        Returns (ms per step of the median round, mean context during that round, kernels launched in it, ms per
        step of every round)."""
        ids = [f"d{batch}-{i}" for i in range(batch)]
        start = ctx - warmup - rounds * steps
        portions = [0]
        for i in ids:
            runner.cache.open(i)
            runner.cache.reserve(i, 0, start)
            runner.cache.commit(i, start)

        def one_step():
            segs = [Segment(i, [1 + k], runner.cache.length(i), [0]) for k, i in enumerate(ids)]
            if args.mixed_chunk:
                portions[0] += 1
                rid = f"portion{portions[0]}"
                runner.cache.open(rid)
                runner.cache.reserve(rid, 0, 1024)
                runner.cache.commit(rid, 1024)
                segs.insert(0, Segment(rid, list(range(1, args.mixed_chunk + 1)), 1024, []))
            logits = runner.step(segs)
            ops.argmax(logits, out_tok[:batch])
            if args.mixed_chunk:
                runner.finish(segs[0].request)

        for _ in range(warmup):
            one_step()
        times, launched = [], 0
        for _ in range(rounds):
            torch.cuda.synchronize()
            before = ops.launch_count
            s, e = events()
            s.record()
            for _ in range(steps):
                one_step()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) / steps)
            launched = ops.launch_count - before
        for i in ids:
            runner.finish(i)
        order = sorted(range(rounds), key=lambda r: times[r])
        mid = order[rounds // 2]
        # the median round ran steps [mid * steps, (mid + 1) * steps) of the timed ones: its mean context
        mean_ctx = ctx - (rounds - mid) * steps + steps / 2.0
        return times[mid], mean_ctx, launched, times

    def decode_bytes(batch: int, context: float) -> float:
        return nums["weight_bytes"] + batch * context * nums["kv_bytes_per_token"]

    if args.prefill_only:
        g = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
        for i in range(max(1, args.steps)):
            s, e = events()
            s.record()
            runner.step([Segment(f"p{i}", prompt, 0, [PREFILL_TOKENS - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.finish(f"p{i}")
            print(json.dumps({"prefill_ms": round(s.elapsed_time(e), 3)}))
        return 0

    # ---- the headline: decode at the default batch, clocks sampled meanwhile -------------------------------
    clocks = ClockSampler()
    clocks.start()
    ms_step, mean_ctx, launches, round_ms = decode_device_timed(args.batch, args.steps, args.warmup, max(1, args.rounds))
    clock_record = clocks.stop()
    clock_record["rounds_ms_per_step"] = [round(t, 4) for t in round_ms]
    value = args.batch * 1000.0 / ms_step
    achieved = decode_bytes(args.batch, mean_ctx) / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                "bytes": int(decode_bytes(args.batch, mean_ctx))}

    # ---- prefill of one 2,048-token prompt ---------------------------------------------------------------------
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()

    def prefill_once(tag):
        s, e = events()
        s.record()
        runner.step([Segment(tag, prompt, 0, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        runner.finish(tag)
        return s.elapsed_time(e)

    # 4 warm-up prefills, then the median of 9: a single 30 ms prefill follows the clock of the moment
    times = [prefill_once(f"p{i}") for i in range(13)] if not args.skip_prefill else [float("nan")] * 13
    pre_ms = statistics.median(times[4:])
    flops = 2.0 * nums["layer_params"] * args.layers * PREFILL_TOKENS + nums["attn_flops_per_layer"](PREFILL_TOKENS) \
        * args.layers + 2.0 * nums["head_params"]
    prefill = {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / pre_ms / 1e9, 1),
               "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}
    if "bf16_tflops_sustained" in pk:       # the same against what the GEMM library sustains under the power cap
        prefill["frac_of_sustained"] = round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    if args.skip_prefill:
        prefill = None

    # ---- decode at batch 1 and 64 --------------------------------------------------------------------------------
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms_b, ctx_b, _, _ = decode_device_timed(b, max(8, args.steps // 2), 3, 3)
            gbs = decode_bytes(b, ctx_b) / (ms_b * 1e-3) / 1e9
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
            points[f"decode_b{b}_ms"] = round(ms_b, 4)
            points[f"decode_b{b}_hbm_frac"] = round(gbs / pk["hbm_gbs"], 4)

    # ---- end to end through the public entry point --------------------------------------------------------------
    e2e = None
    if not args.skip_e2e:
        e2e = end_to_end(engine, args.batch, args.steps, args.warmup, cfg["vocab_size"])
        if not args.skip_points:
            for b in (1, 64):
                other = end_to_end(engine, b, args.steps, args.warmup, cfg["vocab_size"])
                points[f"e2e_b{b}"] = other["value"]

    record = {
        "metric": (f"decode tok/s @ batch {args.batch}, context {ctx} (Qwen3-{args.shape.upper()} shape, bf16, random weights"
                   + (f", a {args.mixed_chunk}-row prompt portion in every step)" if args.mixed_chunk else ")")),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02); device-timed cache content synthetic",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": args.layers,
                   "layers_of_config": shape["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": ctx, "page_size": PAGE, "mixed_chunk": args.mixed_chunk, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 (weights {nums['weight_bytes'] / 1e9:.0f} GB per step)",
                   "cuda_graphs": runner.use_graphs},
        "clocks": clock_record, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "check": check,
    }
    print(json.dumps(record))
    return 0


def end_to_end(engine, batch: int, steps: int, warmup: int, vocab: int):
    """Decode tokens per second through Engine.add_request / Engine.step_once: every step copies its batch
    tables from pinned host memory to the device and reads the sampled tokens back to the host."""
    import torch

    from jllm_serve_b200.sampling import SamplingParams
    # the prompts are prefilled one after the other (two portions each): a request that is ready early decodes while the
    # others' prompts still run, so every request may generate that many tokens more than the timed steps need and none
    # ends inside the timed region
    slack = 2 * batch + 2
    new_tokens = warmup + steps + 1 + slack
    prompt_len = CONTEXT - new_tokens
    g = torch.Generator().manual_seed(2)
    params = SamplingParams.greedy_params(max_tokens=new_tokens, ignore_eos=True)
    ids = [engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), params)
           for _ in range(batch)]
    sched = engine.scheduler
    while any(r.remaining > 1 or not r.output for r in sched.running + sched.waiting):
        engine.step_once()                       # prefill (untimed): until every request is decoding
    for _ in range(warmup - 1):
        engine.step_once()
    torch.cuda.synchronize()
    h2d = engine.runner.builder.bytes_per_step(batch)
    mine = [r for r in sched.running + sched.waiting]

    def generated():
        return sum(len(r.output) for r in mine)

    before = generated()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step_once()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    done = generated() - before          # tokens that were really sampled (a preempted request decodes nothing)
    if done != steps * batch:
        print(f"bench: end to end at batch {batch}: {done} tokens in {steps} steps, expected {steps * batch}",
              file=sys.stderr, flush=True)
    engine.run_until_done()
    for i in ids:
        engine.take_result(i)
    return {"value": round(done / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * engine.sampler.max_rows,
            "ms_per_step": round(dt / steps * 1e3, 4), "tokens_per_step": round(done / steps, 2),
            "preemptions": sched.preemptions}


if __name__ == "__main__":
    sys.exit(main())
