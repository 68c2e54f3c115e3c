"""Decode-phase profiler for the generation engine.

    python -m rl_b200.engine.profile_decode --model llama3.1-8b --batch 64 --context 768 --steps 64 [--layers N] [--eager]

Builds a random-init model, prefills ``batch`` prompts of ``context`` tokens, decodes ``steps`` tokens and prints the
wall time per decode step (host + device) and, from CUDA events around graph replays, the device time per step. Run it
under ``ncu --metrics gpu__time_duration.sum`` with ``--eager --layers 4`` to list every kernel of a decode step.
"""

from __future__ import annotations

import argparse
import json
import time

import torch

from rl_b200.engine.engine import GenerationEngine, SamplingParams
from rl_b200.models.config import preset
from rl_b200.models.transformer import CausalLM


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=768)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--distinct-prompts", action="store_true", help="no prefix sharing between the prompts")
    ap.add_argument("--trace", type=int, default=0, help="after the timed run, trace this many decode windows with the CUDA "
                    "activity profiler and print, per kernel, the mean duration and the mean gap to the kernel before it "
                    "(shares only: durations taken under a profiler are not benchmark figures)")
    ap.add_argument("--trace-out", default="", help="write the traced (kernel, start us, duration us) list to this JSON file")
    ap.add_argument("--quantization", default="", help="mxfp8 | fp8: serve quantised copies of the linear weights (low-precision rollout)")
    a = ap.parse_args(argv)
    mc = preset(a.model)
    if a.layers:
        mc.num_hidden_layers = a.layers
    dev = torch.device("cuda", 0)
    model = CausalLM(mc, dtype=torch.bfloat16, device=dev, seed=0)
    eng = GenerationEngine(model, block_size=64, kv_cache_tokens=a.batch * (a.context + a.steps + 64), max_running=max(64, a.batch),
                           max_model_len=a.context + a.steps + 64, use_cuda_graphs=not a.eager, quantization=a.quantization or None)
    quant = eng.requantize()
    g = torch.Generator().manual_seed(0)
    n_unique = a.batch if a.distinct_prompts else max(1, a.batch // 8)
    uniq = [torch.randint(0, mc.vocab_size, (a.context,), generator=g).tolist() for _ in range(n_unique)]
    prompts = [uniq[i % n_unique] for i in range(a.batch)]
    sp = SamplingParams(max_new_tokens=a.steps, stop_token_ids=[], seed=1)
    eng.generate(prompts, SamplingParams(max_new_tokens=4, stop_token_ids=[], seed=1))  # warm-up, graph capture
    eng.sleep(free_kv_cache=False)
    for k in eng.stats:
        eng.stats[k] = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.generate(prompts, sp)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    st = eng.stats
    out = dict(model=a.model, layers=mc.num_hidden_layers, batch=a.batch, context=a.context, steps=st["decode_steps"],
               graphs=not a.eager, quantization=a.quantization or "bf16", quantized_bytes=(quant or {}).get("quantized_bytes"), wall_s=round(wall, 4), prefill_s=round(st["prefill_s"], 4),
               decode_ms_per_step=round(1e3 * st["decode_s"] / max(1, st["decode_steps"]), 4),
               decode_device_ms_per_step=round(1e3 * st.get("decode_device_s", 0.0) / max(1, st["decode_steps"]), 4),
               weight_stream_floor_ms=round(mc.num_parameters() * 2 / 6.5e12 * 1e3, 3))
    print(json.dumps(out), flush=True)
    if a.trace:
        trace_kernels(eng, prompts, a.trace, a.trace_out)


def trace_kernels(eng, prompts, windows: int, out_path: str = "") -> None:
    """Kernel timeline of a few decode windows (graph replays included) from the CUDA activity profiler: per kernel
    name the launches, the mean duration and the mean idle gap between the end of the previous kernel and its start
    (negative: it overlapped its predecessor through programmatic dependent launch)."""
    from collections import defaultdict

    from torch.profiler import ProfilerActivity, profile

    eng.sleep(free_kv_cache=False)
    steps = windows * eng.decode_window
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.generate(prompts, SamplingParams(max_new_tokens=steps + 1, stop_token_ids=[], seed=2))
        torch.cuda.synchronize()
    import os
    import tempfile

    path = os.path.join(tempfile.mkdtemp(prefix="rlb_trace_"), "trace.json")
    prof.export_chrome_trace(path)
    with open(path) as f:
        events = json.load(f)["traceEvents"]
    evs = sorted((e for e in events if e.get("cat") == "kernel"), key=lambda e: e["ts"])
    # keep the decode part: drop everything up to the last flash-attention (prefill) kernel
    last_prefill = max((i for i, e in enumerate(evs) if "flash_fwd" in e["name"]), default=-1)
    evs = evs[last_prefill + 1:]
    import re

    agg = defaultdict(lambda: [0, 0.0, 0.0])
    prev_end = None
    rows = []
    for e in evs:
        st, en = e["ts"], e["ts"] + e["dur"]
        grid = (e.get("args") or {}).get("grid")
        m = re.search(r"(\w+_kernel|\w+Kernel\w*|\w+_kern\w*)", e["name"])
        k = (m.group(1) if m else e["name"][:40]) + f" grid={grid[0] if grid else '?'}"
        # kernels launched with programmatic dependent launch start (and block) while their predecessor still runs, so the
        # raw duration overstates them: the exclusive time is what the kernel adds after its predecessor has ended
        excl = en - max(st, prev_end) if prev_end is not None else en - st
        agg[k][0] += 1
        agg[k][1] += en - st
        agg[k][2] += max(excl, 0.0)
        rows.append((k, st, e["dur"]))
        prev_end = max(prev_end or en, en)
    span = (evs[-1]["ts"] + evs[-1]["dur"] - evs[0]["ts"]) if evs else 0.0
    print(f"traced {len(evs)} kernels over {span / 1e3:.2f} ms ({steps} decode steps requested)")
    for k, (n, dur, excl) in sorted(agg.items(), key=lambda kv: -kv[1][2]):
        print(f"{k:56s} n={n:6d} mean_us={dur / n:8.2f} exclusive_us={excl / n:8.2f} share={excl / max(span, 1e-9):6.3f}")
    if out_path:
        with open(out_path, "w") as f:
            json.dump(rows[:20000], f)

if __name__ == "__main__":
    main()
