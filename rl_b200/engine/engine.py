"""In-house generation engine: paged KV cache, continuous batching, prompt-prefix sharing between the samples of one
prompt, CUDA-graph decode, temperature / top-k / top-p sampling with per-token log-probabilities.

The host-side scheduler and block manager are C++ (``rl_b200/csrc/engine.cpp``); the forward pass reuses the policy
model's own parameters (the engine holds *views* of the trainer's flat bf16 buffer when colocated at TP1, so a weight
refit is a pointer hand-off) and runs on this repository's kernels. It fills the role that vLLM / SGLang / the mcore
DynamicInferenceEngine play in the reference (nemo_rl/models/generation/vllm/vllm_worker.py:850-1074).

Token accounting: after a prompt of P tokens is prefilled the cache holds P tokens; the first sampled token enters
the cache when the next decode step processes it. A decode step feeds each running sequence's last token at
position ``n = cached tokens``, writes its K/V into slot n and attends over n + 1 tokens.
"""

from __future__ import annotations

import os
import ctypes as C
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from rl_b200.models.transformer import CausalLM, PackedBatch
from rl_b200.ops import engine_ops as E
from rl_b200.ops import functional as F
from rl_b200.ops import lib as _L
from rl_b200.parallel.tensor import gather_cols, row_linear

_P, _I, _LL = C.c_void_p, C.c_int, C.c_longlong
_ENGINE_SIGS = {
    "rlb_engine_create": ([_I, _I, _I, _I], C.c_void_p),
    "rlb_engine_destroy": ([_P], None),
    "rlb_engine_num_free_blocks": ([_P], _I),
    "rlb_engine_num_running": ([_P], _I),
    "rlb_engine_num_waiting": ([_P], _I),
    "rlb_engine_num_preemptions": ([_P], _LL),
    "rlb_engine_add": ([_P, _LL, _I, _I, _LL], _I),
    "rlb_engine_schedule": ([_P, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), C.POINTER(_I)], _I),
    "rlb_engine_get_lists": ([_P, _P, _P, _P, _P, _P], None),
    "rlb_engine_fill_tables": ([_P, _P, _I, _I, _P, _P, _P], _I),
    "rlb_engine_fill_slots": ([_P, _LL, _I, _I, _P], _I),
    "rlb_engine_commit": ([_P, _P, _I, _P], _I),
    "rlb_engine_commit_first": ([_P, _P, _I, _P], _I),
    "rlb_engine_reset": ([_P], None),
    "rlb_engine_set_lookahead": ([_P, _I], None),
    "rlb_engine_window": ([_P], _I),
    "rlb_engine_commit_n": ([_P, _P, _I, _P, _P], _I),
    "rlb_engine_set_hashes": ([_P, _LL, _P, _I], _I),
    "rlb_engine_cached_prefix": ([_P, _LL], _I),
    "rlb_engine_register_prefix": ([_P, _LL], _I),
    "rlb_engine_cache_stats": ([_P, _P, _P, _P, _P], None),
}
_bound = False


def _bind():
    global _bound
    lib = _L.lib()
    if not _bound:
        for name, (args, res) in _ENGINE_SIGS.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res
        _bound = True
    return lib


class _PyScheduler:
    """Pure-Python twin of the C++ scheduler (same rules), used when the native library is not built (CPU tests)."""

    def __init__(self, num_blocks, block_size, max_running, max_prefill_tokens):
        self.nb, self.bs, self.max_running = num_blocks, block_size, max_running
        self.max_prefill = max_prefill_tokens if max_prefill_tokens > 0 else 1 << 30
        self.reset()

    def reset(self):
        self.free = list(range(self.nb - 1, -1, -1))
        self.ref = [0] * self.nb
        self.seqs: dict[int, dict] = {}
        self.waiting: list[int] = []
        self.running: list[int] = []
        self.clock = 0
        self.n_preempt = 0

    def _blocks_for(self, t):
        return (t + self.bs - 1) // self.bs

    def _alloc(self):
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def _release(self, s):
        for b in s["blocks"]:
            self.ref[b] -= 1
            if self.ref[b] == 0:
                self.free.append(b)
        s["blocks"] = []

    def _ensure(self, s, tokens):
        need = self._blocks_for(tokens) - len(s["blocks"])
        if need <= 0:
            return True
        if len(self.free) < need:
            return False
        for _ in range(need):
            s["blocks"].append(self._alloc())
        return True

    def add(self, sid, prompt_len, max_new, share_with):
        if sid in self.seqs or prompt_len <= 0 or self._blocks_for(prompt_len + max_new) > self.nb:
            return -1
        self.seqs[sid] = dict(id=sid, prompt_len=prompt_len, max_new=max_new, num_tokens=0, num_generated=0, running=False,
                              share_with=share_with, prefilled=False, arrival=self.clock, blocks=[])
        self.clock += 1
        self.waiting.append(sid)
        return 0

    def schedule(self):
        prefill, shared, copies = [], [], []
        self.running.sort(key=lambda i: self.seqs[i]["arrival"])
        i = 0
        while i < len(self.running):
            s = self.seqs[self.running[i]]
            if self._ensure(s, s["num_tokens"] + 1):
                i += 1
                continue
            vid = self.running.pop()
            v = self.seqs[vid]
            self._release(v)
            v.update(running=False, prefilled=False, num_tokens=0)
            self.waiting.insert(0, vid)
            self.n_preempt += 1
            if vid == s["id"]:
                break
        decode = list(self.running)
        ptoks = 0
        while self.waiting and len(self.running) < self.max_running:
            sid = self.waiting[0]
            s = self.seqs[sid]
            context = s["prompt_len"] + s["num_generated"]
            partner = None
            if s["share_with"] >= 0 and s["num_generated"] == 0:
                p = self.seqs.get(s["share_with"])
                if p and p["running"] and p["prefilled"] and p["prompt_len"] == s["prompt_len"] and len(p["blocks"]) >= self._blocks_for(s["prompt_len"]):
                    partner = p
            if partner:
                full = s["prompt_len"] // self.bs
                total = self._blocks_for(s["prompt_len"] + 1)
                if len(self.free) < total - full:
                    break
                for b in range(full):
                    s["blocks"].append(partner["blocks"][b])
                    self.ref[partner["blocks"][b]] += 1
                for b in range(full, total):
                    s["blocks"].append(self._alloc())
                if s["prompt_len"] % self.bs:
                    copies.append((partner["blocks"][full], s["blocks"][full]))
                s.update(num_tokens=s["prompt_len"], prefilled=True, running=True)
                shared.append(sid)
            else:
                if ptoks > 0 and ptoks + context > self.max_prefill:
                    break
                if not self._ensure(s, context + 1):
                    break
                ptoks += context
                s.update(num_tokens=context, prefilled=True, running=True)
                prefill.append(sid)
            self.running.append(sid)
            self.waiting.pop(0)
        return prefill, shared, decode, copies

    def tables(self, ids, max_blocks):
        bt = torch.zeros((len(ids), max_blocks), dtype=torch.int32)
        ctx = torch.zeros(len(ids), dtype=torch.int32)
        slots = torch.full((len(ids),), -1, dtype=torch.int64)
        for i, sid in enumerate(ids):
            s = self.seqs[sid]
            nb = len(s["blocks"])
            bt[i, :nb] = torch.tensor(s["blocks"], dtype=torch.int32)
            ctx[i] = s["num_tokens"]
            blk = s["num_tokens"] // self.bs
            if blk < nb:
                slots[i] = s["blocks"][blk] * self.bs + s["num_tokens"] % self.bs
        return bt, ctx, slots

    def slots(self, sid, first, count):
        s = self.seqs[sid]
        return torch.tensor([s["blocks"][(first + t) // self.bs] * self.bs + (first + t) % self.bs for t in range(count)], dtype=torch.int64)

    def commit(self, ids, finished, first=False):
        out = list(finished)
        for i, sid in enumerate(ids):
            s = self.seqs.get(sid)
            if s is None:
                continue
            if not first:
                s["num_tokens"] += 1
            s["num_generated"] += 1
            done = out[i] != 0
            if not done and s["num_generated"] >= s["max_new"]:
                done = True
                out[i] = 2
            if done:
                self._release(s)
                self.running.remove(sid)
                del self.seqs[sid]
        return out

    @property
    def num_free_blocks(self):
        return len(self.free)

    @property
    def num_preemptions(self):
        return self.n_preempt

    def idle(self):
        return not self.waiting and not self.running


class _NativeScheduler:
    """ctypes front of the C++ scheduler."""

    def __init__(self, num_blocks, block_size, max_running, max_prefill_tokens):
        self.lib = _bind()
        self.h = self.lib.rlb_engine_create(num_blocks, block_size, max_running, max_prefill_tokens)
        if not self.h:
            raise RuntimeError("engine creation failed")
        self.bs = block_size

    def __del__(self):
        try:
            if self.h:
                self.lib.rlb_engine_destroy(self.h)
        except Exception:
            pass

    def reset(self):
        self.lib.rlb_engine_reset(self.h)

    def add(self, sid, prompt_len, max_new, share_with):
        return self.lib.rlb_engine_add(self.h, sid, prompt_len, max_new, share_with)

    def schedule(self):
        n = [_I(0) for _ in range(4)]
        self.lib.rlb_engine_schedule(self.h, *[C.byref(x) for x in n])
        npf, nsh, ndc, ncp = (x.value for x in n)
        pf = (_LL * max(npf, 1))()
        sh = (_LL * max(nsh, 1))()
        dc = (_LL * max(ndc, 1))()
        cs = (_I * max(ncp, 1))()
        cd = (_I * max(ncp, 1))()
        self.lib.rlb_engine_get_lists(self.h, pf, sh, dc, cs, cd)
        return list(pf[:npf]), list(sh[:nsh]), list(dc[:ndc]), list(zip(cs[:ncp], cd[:ncp]))

    def tables(self, ids, max_blocks, out=None):
        n = len(ids)
        if out is None:
            bt = torch.empty((n, max_blocks), dtype=torch.int32)
            ctx = torch.empty(n, dtype=torch.int32)
            slots = torch.empty(n, dtype=torch.int64)
        else:
            bt, ctx, slots = out
        arr = (_LL * n)(*ids)
        rc = self.lib.rlb_engine_fill_tables(self.h, arr, n, max_blocks, bt.data_ptr(), ctx.data_ptr(), slots.data_ptr())
        if rc:
            raise RuntimeError(f"fill_tables failed ({rc}): a sequence outgrew max_blocks={max_blocks}")
        return bt, ctx, slots

    def slots(self, sid, first, count):
        out = torch.empty(count, dtype=torch.int64)
        rc = self.lib.rlb_engine_fill_slots(self.h, sid, first, count, out.data_ptr())
        if rc:
            raise RuntimeError(f"fill_slots failed ({rc})")
        return out

    def commit(self, ids, finished, first=False):
        n = len(ids)
        arr = (_LL * n)(*ids)
        fin = (_I * n)(*[int(x) for x in finished])
        (self.lib.rlb_engine_commit_first if first else self.lib.rlb_engine_commit)(self.h, arr, n, fin)
        return list(fin)

    def set_lookahead(self, steps: int) -> None:
        self.lib.rlb_engine_set_lookahead(self.h, int(steps))

    # prefix cache (content-hashed prompt blocks kept across requests and generate calls)
    def set_hashes(self, sid: int, hashes: list[int]) -> None:
        arr = (C.c_ulonglong * max(1, len(hashes)))(*[h & 0xFFFFFFFFFFFFFFFF for h in hashes])
        self.lib.rlb_engine_set_hashes(self.h, sid, arr, len(hashes))

    def cached_prefix(self, sid: int) -> int:
        return max(0, self.lib.rlb_engine_cached_prefix(self.h, sid))

    def register_prefix(self, sid: int) -> int:
        return self.lib.rlb_engine_register_prefix(self.h, sid)

    def cache_stats(self) -> dict:
        v = [_LL(0) for _ in range(4)]
        self.lib.rlb_engine_cache_stats(self.h, *[C.byref(x) for x in v])
        return dict(zip(("hits", "queries", "evictions", "cached_blocks"), (x.value for x in v)))

    @property
    def window(self) -> int:
        return self.lib.rlb_engine_window(self.h)

    def commit_n(self, ids, counts, finished):
        n = len(ids)
        arr = (_LL * n)(*ids)
        cnt = (_I * n)(*[int(x) for x in counts])
        fin = (_I * n)(*[int(x) for x in finished])
        self.lib.rlb_engine_commit_n(self.h, arr, n, cnt, fin)
        return list(fin)

    @property
    def num_free_blocks(self):
        return self.lib.rlb_engine_num_free_blocks(self.h)

    @property
    def num_preemptions(self):
        return self.lib.rlb_engine_num_preemptions(self.h)

    def idle(self):
        return self.lib.rlb_engine_num_running(self.h) == 0 and self.lib.rlb_engine_num_waiting(self.h) == 0


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0  # 0 or None: off
    max_new_tokens: int = 128
    stop_token_ids: Optional[Sequence[int]] = None
    greedy: bool = False
    seed: int = 0


@dataclass
class _Request:
    rid: int
    prompt: list[int]
    max_new: int
    out_tokens: list[int] = field(default_factory=list)
    out_logprobs: list[float] = field(default_factory=list)
    finished: bool = False
    truncated: bool = False
    share_with: int = -1
    uid: int = 0  # keys the request's random stream: same uid and seed -> same draws on any rank / batch
    mm: object = None  # (image patch rows, patches per image) of a vision-language prompt
    routed_experts: object = None  # [prompt + generated tokens, MoE layers, top-k] int16 expert ids (-1: position never ran)


class GenerationEngine:
    """Generates continuations for batches of token prompts with the model's current weights."""

    BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)
    MAX_STOP_IDS = 256   # stop token ids checked on the device after every decode step
    BASE_SEED = 0x5EED   # constant sampler seed; what varies per call and per request travels in the row keys

    @staticmethod
    def _row_key(r, sp) -> int:
        """Random-stream key of a request's next token: call seed (20 bits) | request uid | position (20 bits). The
        decode kernels add one per generated token, so consecutive tokens of a request get consecutive keys."""
        return (((int(sp.seed) * 0x9E3779B1) & 0xFFFFF) << 43) ^ ((int(r.uid) << 20) | len(r.out_tokens))

    def __init__(self, model: CausalLM, *, block_size: int = 64, num_blocks: Optional[int] = None,
                 kv_cache_tokens: Optional[int] = None, gpu_memory_utilization: float = 0.5, max_running: int = 512,
                 max_prefill_tokens: int = 16384, max_model_len: int = 8192, use_cuda_graphs: bool = True,
                 logits_fp32: bool = True, tokenizer=None, quantization: Optional[str] = None, decode_window: int = 16,
                 enable_prefix_caching: bool = True):
        """``quantization``: None (bf16), ``"mxfp8"`` or ``"fp8"``: serve quantised copies of the linear weights
        (see ``engine/quantized.py``); call :meth:`requantize` after the weights changed."""
        self.model = model
        self.quantization = quantization if quantization not in (None, "", "bfloat16", "bf16", "none") else None
        self.cfg = model.cfg
        self.device = model.embed_tokens.device
        self.block_size = block_size
        self.max_model_len = max_model_len
        self.max_blocks_per_seq = (max_model_len + block_size - 1) // block_size + 1
        self.max_running = max_running
        self.max_prefill_tokens = max_prefill_tokens
        self.tokenizer = tokenizer
        self.native = self.device.type == "cuda" and _L.available()
        # tensor parallelism: this rank serves Hq/tp query and Hkv/tp key/value heads; every tp rank runs the same
        # scheduler on the same requests and samples the same tokens (rank 0's sample is broadcast each step)
        self.tp = getattr(model, "tp", None)
        self.tpw = self.tp.world if self.tp is not None else 1
        # hybrid state-space models (Nemotron-H): only the attention blocks have key / value pages; every running sequence
        # also owns one row of each Mamba block's state pools (the last conv inputs and the state-space state), see
        # ``_hybrid_block``. Prefixes are not shared between sequences (pages carry no state) and decode runs eagerly.
        self.hybrid = bool(self.cfg.is_hybrid)
        self._attn_layers = [i for i, l in enumerate(model.layers) if l.self_attn is not None]
        if self.hybrid:
            ep_h = getattr(model, "ep", None)
            if self.tpw > 1 or (ep_h is not None and ep_h.world > 1):
                raise NotImplementedError("the generation engine serves hybrid state-space models on one GPU per replica")
            if self.quantization:
                raise NotImplementedError("quantised rollout is not available for hybrid state-space models")
        # rollout routing replay: when switched on (``record_routing``), every MoE layer reports the experts it chose and the
        # engine files them by request and position; decode then runs eagerly with a host visit per step
        self.record_routing = False
        self._r3_meta = None
        self._r3_buf: list = []
        self.mamba_conv: Optional[list] = None
        self.mamba_ssm: Optional[list] = None
        self._state_row: dict[int, int] = {}
        self._free_rows: list[int] = []
        self._decode_rows: Optional[torch.Tensor] = None
        attn0 = model.layers[self._attn_layers[0]].self_attn if self._attn_layers else None
        self.hq = attn0.hq if attn0 is not None else self.cfg.num_attention_heads
        self.hkv = attn0.hkv if attn0 is not None else self.cfg.num_key_value_heads
        # tensor-parallel decode is captured too when the fused GEMM + all-reduce kernel (device-resident epoch) carries the
        # collectives; NCCL broadcasts / all-gathers of the sampled tokens and logits are capturable as well
        # mixture-of-experts decode is captured as well: its few-token layer (csrc/moe_decode.cu) has fixed shapes and no
        # host visit, on one GPU or, with the peer-memory expert-parallel communicator, across the expert group
        ep0 = getattr(model, "ep", None)
        moe_ok = (not self.cfg.is_moe) or ep0 is None or ep0.world == 1 or getattr(ep0, "comm", None) is not None
        self.use_graphs = use_cuda_graphs and self.native and moe_ok and (self.tpw == 1 or getattr(self.tp, "comm", None) is not None) \
            and not self.hybrid
        self.logits_dtype = torch.float32 if logits_fp32 else model.dtype
        c = self.cfg
        if num_blocks is None:
            if kv_cache_tokens is not None:
                num_blocks = (kv_cache_tokens + block_size - 1) // block_size + max_running
            elif self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                per_block = 2 * max(1, len(self._attn_layers)) * self.hkv * block_size * c.head_dim * 2
                num_blocks = max(16, int(free * gpu_memory_utilization) // per_block)
            else:
                num_blocks = 256
        self.num_blocks = int(num_blocks)
        self.k_cache: Optional[list[torch.Tensor]] = None
        self.v_cache: Optional[list[torch.Tensor]] = None
        sched_cls = _NativeScheduler if _L.available() else _PyScheduler
        self.sched = sched_cls(self.num_blocks, block_size, max_running, max_prefill_tokens)
        # Multi-step decode (native path): the step inputs live on the device and a small kernel advances them after
        # sampling, so the host visits only every `decode_window` steps (one upload of the tables, that many graph
        # replays, one download of the window's tokens). 1 restores a host visit per step.
        self.decode_window = max(1, int(os.environ.get("RLB_DECODE_WINDOW", decode_window))) if self.native else 1
        if self.decode_window > 1 and isinstance(self.sched, _NativeScheduler):
            self.sched.set_lookahead(self.decode_window)
        # Prefix cache: full prompt blocks stay addressable by the hash of the token prefix they end, across requests and
        # generate calls (until the weights change: ``sleep`` resets it). A later prompt with the same prefix, e.g. the next
        # turn of a multi-turn rollout, prefills only its new tokens.
        self.prefix_caching = bool(enable_prefix_caching) and isinstance(self.sched, _NativeScheduler) and not self.hybrid
        self._graphs: dict[int, tuple] = {}
        self._agreed_bucket = 0
        self._static: Optional[dict] = None
        self._step_counter = 0
        self._n_stop = 0
        self.window_hook = None   # optional callable run at every host visit of the generate loop
        # continuous admission (the serving frontend's asynchronous loop): ``admit_hook()`` is asked at every host visit for new
        # requests ``(prompt, max_new_tokens or None, uid, tag)`` that join the running batch; ``finish_hook(request)`` is told
        # the moment a request is complete, long before the generate call returns
        self.admit_hook = None
        self.finish_hook = None
        self.stats = dict(prefill_tokens=0, cached_prefix_tokens=0, decode_steps=0, generated_tokens=0, prefill_s=0.0, decode_s=0.0)
        # optional scheduler timeline: (seconds since the generate call began, sequences decoding, sequences prefilled this
        # iteration, requests not yet finished) per engine iteration, for in-flight batch-size plots
        self._ev = ([torch.cuda.Event(enable_timing=True) for _ in range(2)]
                    if (self.device.type == "cuda" and os.environ.get("RLB_ENGINE_DEVICE_TIME", "0") == "1") else None)
        self._ev_pending = False
        self.stats["decode_device_s"] = 0.0
        self.collect_timeline = False
        self.timeline: list[tuple[float, int, int, int]] = []
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 1
        img = getattr(self.cfg, "image_token_id", None)
        self._banned_ids = torch.tensor([int(img)], dtype=torch.long, device=self.device) if img is not None else None

    def requantize(self) -> Optional[dict]:
        """Refreshes the quantised weight copies from the (refitted) bf16 weights; no-op for a bf16 engine."""
        if not self.quantization:
            return None
        if getattr(self, "quantized_by_refit", False):   # the refit pass already left quantised copies on the weights
            self.quantized_by_refit = False
            return dict(tensors=0, by_refit=True)
        from .quantized import quantize_model

        assert self.tpw == 1, "low-precision rollout with a tensor-parallel engine is not supported"
        return quantize_model(self.model, self.quantization)

    # ------------------------------------------------------------------ memory
    def wake(self) -> None:
        """Allocates the KV cache (no-op when it is resident)."""
        if self.k_cache is not None:
            return
        c = self.cfg
        shape = (self.num_blocks, self.hkv, self.block_size, c.head_dim)
        dt = self.model.dtype
        attn = set(self._attn_layers)
        self.k_cache = [torch.zeros(shape, dtype=dt, device=self.device) if i in attn else None for i in range(len(self.model.layers))]
        self.v_cache = [torch.zeros(shape, dtype=dt, device=self.device) if i in attn else None for i in range(len(self.model.layers))]
        if self.hybrid:   # row 0 is scratch (padding rows of a decode batch write there)
            R = self.max_running + 1
            self.mamba_conv = [torch.zeros((R, c.mamba_conv_dim, c.mamba_d_conv - 1), dtype=dt, device=self.device) if l.kind == "mamba" else None
                               for l in self.model.layers]
            self.mamba_ssm = [torch.zeros((R, c.mamba_num_heads, c.mamba_head_dim, c.ssm_state_size), dtype=torch.float32, device=self.device)
                              if l.kind == "mamba" else None for l in self.model.layers]
            self._state_row, self._free_rows = {}, list(range(R - 1, 0, -1))

    def sleep(self, free_kv_cache: bool = True) -> None:
        """Ends a generation phase: drops all requests; optionally returns the KV cache memory (captured graphs are
        tied to the cache addresses and are dropped with it)."""
        self.sched.reset()
        if self.hybrid:
            self._state_row, self._free_rows = {}, list(range(self.max_running, 0, -1))
        if free_kv_cache:
            self._graphs.clear()
            self._static = None
            self.k_cache = self.v_cache = None
            self.mamba_conv = self.mamba_ssm = None
            if self.device.type == "cuda":
                torch.cuda.empty_cache()

    def kv_cache_bytes(self) -> int:
        c = self.cfg
        return 2 * len(self._attn_layers) * self.num_blocks * self.hkv * self.block_size * c.head_dim * self.model.dtype.itemsize if hasattr(self.model.dtype, "itemsize") else 0

    # ------------------------------------------------------------------ routed-expert recording (rollout routing replay)
    def set_record_routing(self, on: bool) -> None:
        moe = [l.mlp for l in self.model.layers if getattr(l, "mlp", None) is not None and hasattr(l.mlp, "routing_sink")]
        self.record_routing = bool(on) and bool(moe)
        for j, m in enumerate(moe):
            m._r3_layer = j
            m.routing_sink = self._r3_sink if self.record_routing else None
        self._r3_layers = len(moe)

    def _r3_sink(self, moe, idx) -> None:
        meta = self._r3_meta
        if meta is None:
            return
        n = meta[0].numel()
        self._r3_buf.append((moe._r3_layer, meta[0], meta[1], idx[:n].to(torch.int16)))

    def _r3_rows(self, sids, positions) -> None:
        """Declares which (request, position) every row of the next forward pass is."""
        if self.record_routing:
            self._r3_meta = (torch.as_tensor(sids, dtype=torch.int64), torch.as_tensor(positions, dtype=torch.int64).cpu())

    def _r3_assemble(self, reqs: dict) -> None:
        buf, self._r3_buf, self._r3_meta = self._r3_buf, [], None
        if not buf or not reqs:
            return
        k = buf[0][3].shape[1]
        start, total = {}, 0
        for sid, r in reqs.items():
            start[sid] = total
            total += len(r.prompt) + len(r.out_tokens)
        big = torch.full((total, self._r3_layers, k), -1, dtype=torch.int16)
        base = torch.zeros(max(reqs) + 1, dtype=torch.int64)
        size = torch.zeros(max(reqs) + 1, dtype=torch.int64)
        for sid, r in reqs.items():
            base[sid], size[sid] = start[sid], len(r.prompt) + len(r.out_tokens)
        for layer, sids, pos, idx in buf:      # in issue order: a re-prefilled (preempted) sequence overwrites its rows
            ok = pos < size[sids]
            big[(base[sids] + pos)[ok], layer] = idx.cpu()[ok]
        for sid, r in reqs.items():
            r.routed_experts = big[start[sid] : start[sid] + len(r.prompt) + len(r.out_tokens)]

    # ------------------------------------------------------------------ hybrid state-space models
    def _claim_state_rows(self, live) -> None:
        """Keeps one state row per sequence that is scheduled this iteration and returns the rows of sequences that are not
        (finished, or preempted: a preempted sequence is prefilled again from its first token, which rebuilds its state)."""
        for sid in [s for s in self._state_row if s not in live]:
            self._free_rows.append(self._state_row.pop(sid))
        for sid in live:
            if sid not in self._state_row:
                if not self._free_rows:
                    raise RuntimeError("no free state row: more sequences scheduled than max_running")
                self._state_row[sid] = self._free_rows.pop()

    def _hybrid_block(self, li: int, layer, h, seq=None):
        """A block of a hybrid model that is not attention. ``seq`` = (cu_seqlens, max_len, state rows [sequences]) for whole
        (pieces of) sequences, whose Mamba states start from and are left in the pools; None: one token per sequence of the
        decode batch (``self._decode_rows``)."""
        x = F.rmsnorm(h, layer.norm, self.cfg.rms_norm_eps)
        if layer.kind != "mamba":
            return layer.mlp(x, h)
        conv, ssm = self.mamba_conv[li], self.mamba_ssm[li]
        if seq is None:
            rows = self._decode_rows
            y, c1, s1 = layer.mamba.step(x, conv[rows], ssm[rows])
        else:
            cu, max_len, rows = seq
            y, (c1, s1) = layer.mamba(x, cu, max_len, state=(conv[rows], ssm[rows]), return_state=True)
        conv.index_copy_(0, rows, c1.to(conv.dtype))
        ssm.index_copy_(0, rows, s1)
        return h + y

    def _zero_state_rows(self, rows: torch.Tensor) -> None:
        for cbuf, sbuf in zip(self.mamba_conv, self.mamba_ssm):
            if cbuf is not None:
                cbuf.index_fill_(0, rows, 0)
                sbuf.index_fill_(0, rows, 0)

    # ------------------------------------------------------------------ model forward (inference)
    def _layer_tail(self, layer, h, a):
        # o_proj (tp > 1: GEMM + all-reduce (+ residual) in one kernel; adds LoRA deltas), norms and MLP in the family's order
        return layer.tail(h, a)

    def _embed(self, ids):
        m = self.model
        h = F.embedding(ids, m.embed_tokens)
        s = self.cfg.embed_scale
        return h if s == 1.0 else h * torch.tensor(s, dtype=h.dtype, device=h.device)

    def _freq(self, layer):
        """RoPE frequencies of a layer (sliding-window layers may rotate with their own base)."""
        m = self.model
        if self.cfg.is_mla:   # latent attention rotates its decoupled rotary part itself: the cache write rotates by zero
            if getattr(self, "_zero_freq", None) is None:
                self._zero_freq = torch.zeros(self.cfg.head_dim // 2, dtype=torch.float32, device=self.device)
            return self._zero_freq
        return m.inv_freq_local if (layer.window and m.inv_freq_local is not None) else m.inv_freq

    def _output_logits(self, h, out=None):
        """[n, V] logits: the local vocabulary slice is projected here and the slices are gathered over the tp group."""
        z = F.gemm(h, self.model.output_weight, out=out if self.tpw == 1 else None, out_dtype=self.logits_dtype)
        if self.tpw > 1:
            comm = getattr(self.tp, "comm", None)
            # peer-memory column gather (no NCCL inside the captured decode step); NCCL / gloo twin otherwise
            z = comm.gather_cols(z) if (comm is not None and self.native and z.shape[0] <= 1024) else gather_cols(z, self.tp)
        if self._banned_ids is not None:   # placeholder tokens (image slots) are inputs only: never sampled
            z.index_fill_(1, self._banned_ids, -1e30)
        return z

    def _agree_max(self, ep, values: list[int]) -> list[int]:
        """Element-wise maximum of a few integers over the expert-parallel group (one small all-reduce, one host read)."""
        import torch.distributed as dist

        t = torch.tensor(values, dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ep.group)
        return [int(x) for x in t.tolist()]

    @torch.no_grad()
    def _dummy_forward(self, decode: bool) -> None:
        self._r3_meta = None
        """One forward pass over a single padding token (slot -1: nothing is written to the KV cache)."""
        dev = self.device
        idt = torch.int32 if self.native else torch.int64
        ids = torch.zeros(1, dtype=idt, device=dev)
        pos = torch.zeros(1, dtype=torch.int32, device=dev)
        slots = torch.full((1,), -1, dtype=torch.int64, device=dev)
        if decode:
            bt = torch.zeros((1, self.max_blocks_per_seq), dtype=torch.int32, device=dev)
            self._decode_forward(ids, pos, slots, bt, torch.zeros(1, dtype=torch.int32, device=dev), 1, None)
        else:
            cu = torch.tensor([0, 1], dtype=torch.int32, device=dev)
            self._prefill_forward(PackedBatch(ids, pos, cu, 1), slots, torch.zeros(1, dtype=torch.int64, device=dev))

    def _agree(self, tok, lp):
        """All tp ranks must take the same scheduling decisions. After the logits gather every rank holds bit-identical
        logits (the gather copies, the all-reduce GEMMs sum in a fixed rank order) and the sampler's random stream is keyed
        by (seed, request, position), so every rank draws the same token without talking to the others. The broadcast of
        rank 0's samples is kept as an option (``RLB_TP_AGREE=1``) for back ends whose reductions are not bit-reproducible."""
        if self.tpw > 1 and os.environ.get("RLB_TP_AGREE", "0") == "1":
            import torch.distributed as dist

            src = dist.get_global_rank(self.tp.group, 0) if self.tp.group is not None else 0
            dist.broadcast(tok, src=src, group=self.tp.group)
            dist.broadcast(lp, src=src, group=self.tp.group)
        return tok, lp

    @torch.no_grad()
    def _prefill_forward(self, batch: PackedBatch, slots: torch.Tensor, last_idx: torch.Tensor, state_rows=None) -> torch.Tensor:
        m, c = self.model, self.cfg
        h = self._embed(batch.input_ids)
        if hasattr(m, "merge_vision"):
            h = m.merge_vision(h, batch.input_ids, getattr(batch, "mm", None))
        for li, layer in enumerate(m.layers):
            if self.hybrid and layer.kind != "attention":
                h = self._hybrid_block(li, layer, h, (batch.cu_seqlens, batch.max_seqlen, state_rows))
                continue
            x = F.rmsnorm(h, layer.input_layernorm, c.rms_norm_eps)
            qkv = layer.self_attn.project_qkv(x, batch.positions, m.inv_freq, apply_rope=False)
            qkv = E.rope_kv_cache_write(qkv, batch.positions, self._freq(layer), slots, self.k_cache[li], self.v_cache[li], self.hq, self.hkv, c.head_dim)
            a = F.attention_varlen(qkv, batch.cu_seqlens, batch.max_seqlen, self.hq, self.hkv, c.head_dim, scale=c.attn_scale, window=layer.window)
            h = self._layer_tail(layer, h, a)
        hl = E.gather_rows(h, last_idx.to(torch.int32))
        hl = F.rmsnorm(hl, m.norm, c.rms_norm_eps)
        return self._output_logits(hl)

    def _can_fuse_decode(self, n: int) -> bool:
        """The decode step with RMSNorm and SwiGLU folded into the projections' epilogues (7 kernels per layer instead of
        10) covers dense bf16 layers on one GPU; everything else takes the layer-by-layer path below."""
        c = self.cfg
        if not (self.native and self.tpw == 1 and not self.quantization and not c.is_moe and not self.hybrid and n <= 256
                and os.environ.get("RLB_FUSED_DECODE", "1") != "0"):
            return False
        if c.hidden_size % 128 or c.intermediate_size % 64 or not len(self.model.layers):
            return False
        if c.sandwich_norm or c.hidden_act != "silu" or c.embed_scale != 1.0 or c.sliding_window or c.attn_scale is not None or c.is_mla:
            return False   # the fused step hard-wires the Llama / Qwen block structure
        l0 = self.model.layers[0]
        if any(getattr(p, "_rlb_qat", None) is not None for p in l0.parameters()):
            return False   # quantisation-aware training: the projections go through the quantise-dequantise operators
        return getattr(l0.self_attn, "qkv_lora", None) is None and getattr(l0.mlp, "gate_up_lora", None) is None

    @torch.no_grad()
    def _decode_forward_fused(self, ids, positions, slots, block_table, seq_lens, num_splits, scratch, logits_out=None):
        """Decode step whose norms ride in the GEMM epilogues: the projection that produces the residual stream also
        writes ``h * w_norm`` and per-tile sums of squares, the next projection scales its rows by the reciprocal RMS, and
        gate_up applies SwiGLU itself (``rlb_gemm_skinny_fused``)."""
        m, c = self.model, self.cfg
        eps = c.rms_norm_eps
        n, d = ids.shape[0], c.hidden_size
        tiles = (d + 127) // 128
        dev = ids.device
        hw = torch.empty((n, d), dtype=m.dtype, device=dev)
        hw2 = torch.empty((n, d), dtype=m.dtype, device=dev)
        ssq = torch.empty((tiles, 256), dtype=torch.float32, device=dev)
        ssq2 = torch.empty((tiles, 256), dtype=torch.float32, device=dev)
        h = F.embedding(ids, m.embed_tokens)
        L = len(m.layers)
        for li, layer in enumerate(m.layers):
            at = layer.self_attn
            if li == 0:   # the embedding has no epilogue to leave the statistics: one plain norm per step
                qkv = E.skinny_linear(F.rmsnorm(h, layer.input_layernorm, eps), at.qkv_proj, bias=at.qkv_bias)
            else:
                qkv = E.skinny_linear(hw, at.qkv_proj, bias=at.qkv_bias, ssq_in=ssq, eps=eps)
            if c.qk_norm:
                qkv = F.head_rmsnorm(qkv, at.q_norm, 0, at.hq, c.head_dim, eps)
                qkv = F.head_rmsnorm(qkv, at.k_norm, at.q_local, at.hkv, c.head_dim, eps)
            qkv = E.rope_kv_cache_write(qkv, positions, m.inv_freq, slots, self.k_cache[li], self.v_cache[li], self.hq, self.hkv, c.head_dim)
            a = E.paged_decode(qkv, self.k_cache[li], self.v_cache[li], block_table, seq_lens, self.hq, self.hkv, c.head_dim,
                               num_splits=num_splits, scratch=scratch)
            h = E.skinny_linear(a, at.o_proj, residual=h, ssq_out=ssq2, norm_w=layer.post_attention_layernorm, out2=hw2)
            act = E.skinny_linear(hw2, layer.mlp.gate_up_proj, ssq_in=ssq2, eps=eps, swiglu=True)
            next_w = m.layers[li + 1].input_layernorm if li + 1 < L else m.norm
            h = E.skinny_linear(act, layer.mlp.down_proj, residual=h, ssq_out=ssq, norm_w=next_w, out2=hw)
        z = E.skinny_linear(hw, m.output_weight, out=logits_out, out_dtype=self.logits_dtype, ssq_in=ssq, eps=eps)
        if self._banned_ids is not None:
            z.index_fill_(1, self._banned_ids, -1e30)
        return z

    def _can_fuse_decode_tp(self, n: int) -> bool:
        """Tensor-parallel decode on the weight-streaming GEMM: the row-parallel projections leave fp32 partial sums that a
        one-shot peer all-reduce kernel sums, adds to the residual stream and normalises for the next projection."""
        c = self.cfg
        if not (self.native and self.tpw > 1 and getattr(self.tp, "comm", None) is not None and not self.quantization and not c.is_moe
                and n <= 256 and os.environ.get("RLB_FUSED_DECODE_TP", "1") != "0"):
            return False
        if c.hidden_size % 128 or not len(self.model.layers):
            return False
        if c.sandwich_norm or c.hidden_act != "silu" or c.embed_scale != 1.0 or c.sliding_window or c.attn_scale is not None or c.is_mla:
            return False
        l0 = self.model.layers[0]
        if any(getattr(p, "_rlb_qat", None) is not None for p in l0.parameters()):
            return False
        f_local = l0.mlp.gate_up_proj.shape[0] // 2
        return (f_local % 64 == 0 and getattr(l0.self_attn, "qkv_lora", None) is None and getattr(l0.mlp, "gate_up_lora", None) is None
                and getattr(l0.self_attn, "o_lora", None) is None)

    @torch.no_grad()
    def _decode_forward_fused_tp(self, ids, positions, slots, block_table, seq_lens, num_splits, scratch, logits_out=None):
        """Per layer: qkv (column shard) -> rope + cache write -> paged attention over the local heads -> o_proj partial sums ->
        all-reduce + residual + post-attention norm (one peer kernel) -> gate_up with SwiGLU -> down partial sums ->
        all-reduce + residual + next input norm. No NCCL call: the step is captured in a CUDA graph."""
        m, c, comm = self.model, self.cfg, self.tp.comm
        eps = c.rms_norm_eps
        h = F.embedding(ids, m.embed_tokens)
        L = len(m.layers)
        x = F.rmsnorm(h, m.layers[0].input_layernorm, eps)
        for li, layer in enumerate(m.layers):
            at = layer.self_attn
            qkv = E.skinny_linear(x, at.qkv_proj, bias=at.qkv_bias)
            if c.qk_norm:
                qkv = F.head_rmsnorm(qkv, at.q_norm, 0, at.hq, c.head_dim, eps)
                qkv = F.head_rmsnorm(qkv, at.k_norm, at.q_local, at.hkv, c.head_dim, eps)
            qkv = E.rope_kv_cache_write(qkv, positions, m.inv_freq, slots, self.k_cache[li], self.v_cache[li], self.hq, self.hkv, c.head_dim)
            a = E.paged_decode(qkv, self.k_cache[li], self.v_cache[li], block_table, seq_lens, self.hq, self.hkv, c.head_dim,
                               num_splits=num_splits, scratch=scratch)
            part = E.skinny_linear(a, at.o_proj, out_dtype=torch.float32)
            h, x2 = comm.allreduce_rows(part, h, layer.post_attention_layernorm, eps)
            act = E.skinny_linear(x2, layer.mlp.gate_up_proj, swiglu=True)
            part = E.skinny_linear(act, layer.mlp.down_proj, out_dtype=torch.float32)
            next_w = m.layers[li + 1].input_layernorm if li + 1 < L else m.norm
            h, x = comm.allreduce_rows(part, h, next_w, eps)
        return self._output_logits(x, logits_out)

    @torch.no_grad()
    def _decode_forward(self, ids, positions, slots, block_table, seq_lens, num_splits, scratch, logits_out=None):
        if self._can_fuse_decode(ids.shape[0]):
            return self._decode_forward_fused(ids, positions, slots, block_table, seq_lens, num_splits, scratch, logits_out)
        if self._can_fuse_decode_tp(ids.shape[0]):
            return self._decode_forward_fused_tp(ids, positions, slots, block_table, seq_lens, num_splits, scratch, logits_out)
        m, c = self.model, self.cfg
        h = self._embed(ids)
        for li, layer in enumerate(m.layers):
            if self.hybrid and layer.kind != "attention":
                h = self._hybrid_block(li, layer, h)
                continue
            x = F.rmsnorm(h, layer.input_layernorm, c.rms_norm_eps)
            qkv = layer.self_attn.project_qkv(x, positions, m.inv_freq, apply_rope=False)
            qkv = E.rope_kv_cache_write(qkv, positions, self._freq(layer), slots, self.k_cache[li], self.v_cache[li], self.hq, self.hkv, c.head_dim)
            a = E.paged_decode(qkv, self.k_cache[li], self.v_cache[li], block_table, seq_lens, self.hq,
                               self.hkv, c.head_dim, scale=c.attn_scale, window=layer.window, num_splits=num_splits, scratch=scratch)
            h = self._layer_tail(layer, h, a)
        h = F.rmsnorm(h, m.norm, c.rms_norm_eps)
        return self._output_logits(h, logits_out)

    # ------------------------------------------------------------------ decode step (eager or CUDA graph)
    def _static_buffers(self):
        """Fixed-address inputs and outputs of the decode step. All inputs live in one device blob mirrored by one pinned host
        blob, so a step uploads them with a single copy; the sampled tokens and their log-probabilities share one output blob
        and come back with a single copy."""
        if self._static is None:
            B, MB = self.max_running, self.max_blocks_per_seq
            W = self.decode_window
            dev = self.device
            fields = [("slots", torch.int64, (B,)), ("keys", torch.int64, (B,)), ("ids", torch.int32, (B,)), ("positions", torch.int32, (B,)),
                      ("seq_lens", torch.int32, (B,)), ("active", torch.int32, (B,)), ("remaining", torch.int32, (B,)),
                      ("win_step", torch.int32, (4,)), ("stop_ids", torch.int32, (self.MAX_STOP_IDS,)), ("state_rows", torch.int64, (B,)),
                      ("block_table", torch.int32, (B, MB))]
            offs, total = {}, 0
            for name, dt, shape in fields:
                n = 1
                for x in shape:
                    n *= x
                offs[name] = (total, n * torch.empty((), dtype=dt).element_size(), dt, shape)
                total += -(-offs[name][1] // 16) * 16
            blob = torch.zeros(total, dtype=torch.uint8, device=dev)
            host_blob = torch.zeros(total, dtype=torch.uint8)
            if dev.type == "cuda":
                host_blob = host_blob.pin_memory()
            # outputs of a window: [tokens produced per row | sampled tokens, step-major | their log-probabilities]
            out_blob = torch.zeros(B + 2 * W * B, dtype=torch.int32, device=dev)
            step_out = torch.zeros(2 * B, dtype=torch.int32, device=dev)   # the current step's samples

            def views(buf):
                return {name: buf[o : o + nb].view(dt).view(shape) for name, (o, nb, dt, shape) in offs.items()}

            self._static = dict(views(blob), blob=blob, host_blob=host_blob, host=views(host_blob), out_blob=out_blob,
                                produced=out_blob[:B], out_tok=out_blob[B : B + W * B].view(W, B),
                                out_lp=out_blob[B + W * B :].view(torch.float32).view(W, B),
                                tok=step_out[:B], lp=step_out[B:].view(torch.float32),
                                temps=torch.ones(B, dtype=torch.float32, device=dev), top_ks=torch.zeros(B, dtype=torch.int32, device=dev),
                                top_ps=torch.ones(B, dtype=torch.float32, device=dev))
            self._static["slots"].fill_(-1)
            self._static["host"]["slots"].fill_(-1)
        return self._static

    def _bucket(self, n: int) -> int:
        if self._agreed_bucket:   # expert-parallel ranks decode batches of one size (the largest any of them needs)
            return max(self._agreed_bucket, n)
        for b in self.BUCKETS:
            if b >= n:
                return min(b, self.max_running) if b <= self.max_running else n
        return n

    def _decode_body(self, st, B, sp: SamplingParams, num_splits, scratch):
        self._decode_rows = st["state_rows"][:B]
        logits = self._decode_forward(st["ids"][:B], st["positions"][:B], st["slots"][:B], st["block_table"][:B],
                                      st["seq_lens"][:B], num_splits, scratch)
        E.sample(logits, temperature=sp.temperature, top_k=sp.top_k or 0, top_p=sp.top_p, greedy=sp.greedy, seed=self.BASE_SEED,
                 row_keys=st["keys"][:B], out=(st["tok"][:B], st["lp"][:B]))
        self._agree(st["tok"][:B], st["lp"][:B])
        if self.native:
            E.decode_advance(st, B, self.block_size, self.decode_window, self._n_stop)
        return logits

    def _run_decode(self, n: int, sp: SamplingParams, max_ctx: int, steps: int = 1):
        """Runs ``steps`` decode steps back to back from the device-resident step inputs (native path)."""
        st = self._static_buffers()
        B = self._bucket(n)
        c = self.cfg
        num_splits = E.choose_splits(B, self.hkv, max(self.max_model_len // 2, 1), self.block_size, self._sm_count) if self.native else 1
        if not self.native:
            self._decode_rows = st["state_rows"][:n]
            logits = self._decode_forward(st["ids"][:n].long(), st["positions"][:n], st["slots"][:n], st["block_table"][:n],
                                          st["seq_lens"][:n], 1, None)
            tok, lp = E.sample(logits, temperature=sp.temperature, top_k=sp.top_k or 0, top_p=sp.top_p, greedy=sp.greedy,
                               seed=self.BASE_SEED, row_keys=st["keys"][:n])
            tok, lp = self._agree(tok, lp)
            return tok[:n], lp[:n]
        # the per-call seed is not part of the key: it reaches the sampler through the row keys (device memory), so one
        # captured graph serves every generate call with the same sampling parameters
        key = (B, num_splits, sp.temperature, sp.top_k or 0, sp.top_p, sp.greedy, self._n_stop)
        use_graphs = self.use_graphs and not self.record_routing
        ep = getattr(self.model, "ep", None)
        if c.is_moe:
            # the few-token MoE layer needs every expert-parallel rank to run the same batch size (the generate loop agreed
            # on this bucket); larger batches take the dispatch / combine path, which is not captured
            from rl_b200.ops.moe_ops import SMALL_MAX_COPIES

            W = ep.world if ep is not None else 1
            cap = SMALL_MAX_COPIES // (W * c.num_experts_per_tok)
            fits = B <= min(cap, 256 if W == 1 else cap)
            if W > 1:
                ep.lockstep_max = min(cap, max(self.max_running, B))
                ep.lockstep_tokens = B if (fits and getattr(ep, "comm", None) is not None and self._agreed_bucket) else 0
                fits = ep.lockstep_tokens > 0
            use_graphs = use_graphs and fits
        try:
            return self._run_decode_steps(n, B, sp, num_splits, key, use_graphs, steps, st)
        finally:
            if c.is_moe and ep is not None and ep.world > 1:
                ep.lockstep_tokens = 0

    def _run_decode_steps(self, n, B, sp, num_splits, key, use_graphs, steps, st):
        c = self.cfg
        if use_graphs:
            g = self._graphs.get(key)
            if g is None:
                no, nml = E.decode_scratch_sizes(B, self.hq, num_splits, c.head_dim)
                scratch = (torch.empty(no, dtype=torch.float32, device=self.device), torch.empty(nml, dtype=torch.float32, device=self.device)) if num_splits > 1 else None
                # warm-up outside capture (sets kernel attributes, sizes the allocator), then capture
                side = torch.cuda.Stream(device=self.device)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._decode_body(st, B, sp, num_splits, scratch)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                before = _L.Counters.launches
                with torch.cuda.graph(graph):
                    self._decode_body(st, B, sp, num_splits, scratch)
                g = (graph, scratch, _L.Counters.launches - before)
                self._graphs[key] = g
            if self._ev is not None:   # device time of the replays alone (the window's host work shows as decode_s minus this)
                self._ev[0].record()
            for _ in range(steps):
                g[0].replay()
            if self._ev is not None:
                self._ev[1].record()
                self._ev_pending = True
            _L.Counters.graph_replayed(g[2] * steps)
        else:
            no, nml = E.decode_scratch_sizes(B, self.hq, num_splits, c.head_dim)
            scratch = (torch.empty(no, dtype=torch.float32, device=self.device), torch.empty(nml, dtype=torch.float32, device=self.device)) if num_splits > 1 else None
            for _ in range(steps):
                self._decode_body(st, B, sp, num_splits, scratch)
        return st["tok"][:n], st["lp"][:n]

    def _block_hashes(self, tokens: list[int]) -> list[int]:
        """Chained content hashes of the full blocks of a prompt: entry i identifies tokens [0, (i + 1) * block_size)."""
        bs, out, h = self.block_size, [], 0x9E3779B97F4A7C15
        for i in range(len(tokens) // bs):
            h = hash((h, tuple(tokens[i * bs : (i + 1) * bs]))) & 0xFFFFFFFFFFFFFFFF
            out.append(h)
        return out

    def _prefill_plain(self, items, reqs, dev) -> dict:
        """Whole prompts in one packed batch (nothing cached, nothing longer than the prefill budget)."""
        toks, lens, slots = [], [], []
        for sid, seq, _ in items:
            toks.extend(seq)
            lens.append(len(seq))
            slots.append(self.sched.slots(sid, 0, len(seq)))
        ids = _L.to_device(torch.tensor(toks, dtype=torch.int32 if self.native else torch.int64), dev)
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0)
        pos = torch.cat([torch.arange(L, dtype=torch.int32) for L in lens]).to(dev)
        batch = PackedBatch(ids, pos, cu.to(dev), max(lens))
        mms = [reqs[sid].mm for sid, _, _ in items if getattr(reqs[sid], "mm", None) is not None]
        if mms:
            batch.mm = dict(patches=_L.to_device(torch.cat([m[0] for m in mms]), dev), sizes=[int(x) for m in mms for x in m[1]])
        self._r3_rows([sid for (sid, _, _), L in zip(items, lens) for _ in range(L)], pos)
        rows = None
        if self.hybrid:   # whole prompts: the states start from zero
            rows = torch.tensor([self._state_row[sid] for sid, _, _ in items], dtype=torch.int64, device=dev)
            self._zero_state_rows(rows)
        logits = self._prefill_forward(batch, torch.cat(slots).to(dev), (cu[1:] - 1).to(dev), rows)
        self.stats["prefill_tokens"] += len(toks)
        return {sid: logits[j] for j, (sid, _, _) in enumerate(items)}

    def _prefill_with_prefix(self, items, dev, cap: int) -> dict:
        """Prefill of prompts whose leading tokens are already in the KV cache (prefix-cache hits) and / or that are longer
        than the prefill budget. Only the new tokens go through the projections and MLPs; their attention sees the cached
        prefix through keys / values read back from the cache pages. A long prompt is cut into chunks of at most ``cap``
        tokens that run one after the other, each attending to the chunks before it the same way (chunked prefill)."""
        done = {sid: cached for sid, _, cached in items}
        self.stats["cached_prefix_tokens"] += sum(done.values())
        out: dict = {}
        while True:
            round_items, budget = [], cap
            for sid, seq, _ in items:
                left = len(seq) - done[sid]
                if left <= 0 or budget <= 0:
                    continue
                n = min(left, budget)
                round_items.append((sid, seq, done[sid], n))
                budget -= n
            if not round_items:
                break
            logits = self._prefill_round(round_items, dev)
            for j, (sid, seq, p, n) in enumerate(round_items):
                done[sid] = p + n
                if done[sid] == len(seq):
                    out[sid] = logits[j]
                self.stats["prefill_tokens"] += n
        return out

    @torch.no_grad()
    def _prefill_round(self, round_items, dev) -> torch.Tensor:
        """One packed forward over the NEW tokens of several sequences: sequence i contributes tokens [p_i, p_i + n_i) and
        attends to its p_i cached tokens. Returns the logits of every sequence's last new token."""
        m, c = self.model, self.cfg
        hq, hkv, D = self.hq, self.hkv, c.head_dim
        idt = torch.int32 if self.native else torch.int64
        toks, pos, new_slots, pre_slots, full_lens, new_idx, pre_idx, last = [], [], [], [], [], [], [], []
        row = 0
        for sid, seq, p, n in round_items:
            toks.extend(seq[p : p + n])
            pos.append(torch.arange(p, p + n, dtype=torch.int32))
            new_slots.append(self.sched.slots(sid, p, n))
            if p:
                pre_slots.append(self.sched.slots(sid, 0, p))
                pre_idx.append(torch.arange(row, row + p))
            new_idx.append(torch.arange(row + p, row + p + n))
            row += p + n
            full_lens.append(p + n)
            last.append(len(toks) - 1)
        ids = _L.to_device(torch.tensor(toks, dtype=idt), dev)
        self._r3_rows([sid for sid, _, _, n in round_items for _ in range(n)], torch.cat(pos))
        positions = torch.cat(pos).to(dev)
        slots = torch.cat(new_slots).to(dev)
        new_rows = torch.cat(new_idx).to(dev)
        cu = torch.zeros(len(full_lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(full_lens, dtype=torch.int64).cumsum(0)
        cu = cu.to(dev)
        if pre_slots:
            ps = torch.cat(pre_slots).to(dev)
            pre_rows = torch.cat(pre_idx).to(dev)
            pre_blk, pre_off = ps // self.block_size, ps % self.block_size
        total, W = row, (hq + 2 * hkv) * D
        h = self._embed(ids)
        if self.hybrid:   # the new tokens as sequences of their own; a piece that starts a prompt starts from zero states
            news = [n for _, _, _, n in round_items]
            cu_new = torch.zeros(len(news) + 1, dtype=torch.int32)
            cu_new[1:] = torch.tensor(news, dtype=torch.int64).cumsum(0)
            cu_new = cu_new.to(dev)
            st_rows = torch.tensor([self._state_row[sid] for sid, _, _, _ in round_items], dtype=torch.int64, device=dev)
            fresh = [self._state_row[sid] for sid, _, p, _ in round_items if p == 0]
            if fresh:
                self._zero_state_rows(torch.tensor(fresh, dtype=torch.int64, device=dev))
        for li, layer in enumerate(m.layers):
            if self.hybrid and layer.kind != "attention":
                h = self._hybrid_block(li, layer, h, (cu_new, max(news), st_rows))
                continue
            x = F.rmsnorm(h, layer.input_layernorm, c.rms_norm_eps)
            qkv = layer.self_attn.project_qkv(x, positions, m.inv_freq, apply_rope=False)
            qkv = E.rope_kv_cache_write(qkv, positions, self._freq(layer), slots, self.k_cache[li], self.v_cache[li], hq, hkv, D)
            if pre_slots:
                # rows of the cached prefix carry keys / values from the cache pages (already rotated) and a zero query
                full = torch.zeros((total, W), dtype=qkv.dtype, device=dev)
                full[new_rows] = qkv
                full[pre_rows, hq * D : (hq + hkv) * D] = self.k_cache[li][pre_blk, :, pre_off, :].reshape(-1, hkv * D)
                full[pre_rows, (hq + hkv) * D :] = self.v_cache[li][pre_blk, :, pre_off, :].reshape(-1, hkv * D)
                a = F.attention_varlen(full, cu, max(full_lens), hq, hkv, D, scale=c.attn_scale, window=layer.window)[new_rows]
            else:
                a = F.attention_varlen(qkv, cu, max(full_lens), hq, hkv, D, scale=c.attn_scale, window=layer.window)
            h = self._layer_tail(layer, h, a)
        hl = E.gather_rows(h, torch.tensor(last, dtype=torch.int32, device=dev))
        return self._output_logits(F.rmsnorm(hl, m.norm, c.rms_norm_eps))

    def _window_steps(self, decode, reqs) -> int:
        """How many decode steps the next window may run for these sequences: bounded by the blocks the scheduler reserved
        ahead, the window size and the longest remaining budget."""
        if not decode:
            return 0
        max_rem = max(1, max(reqs[sid].max_new - len(reqs[sid].out_tokens) for sid in decode))
        return max(1, min(self.sched.window if isinstance(self.sched, _NativeScheduler) else 1, self.decode_window, max_rem))

    def _decode_window_native(self, decode, reqs, sp: SamplingParams, stop: set, st, steps: Optional[int] = None) -> None:
        """One window of decode steps for the running sequences: upload the step inputs and block tables once, run up to
        ``decode_window`` steps on the device (each step's sampled token feeds the next through the advance kernel, stop
        tokens and length limits retire rows on the device), then read all tokens of the window with one copy.
        ``steps``: the step count the ranks of an expert-parallel group agreed on (never above this rank's own bound); a
        rank without running sequences takes part with a batch of inactive rows."""
        t0 = time.perf_counter()
        n = len(decode)
        hb = st["host"]
        max_ctx = 1
        if n:
            self.sched.tables(decode, self.max_blocks_per_seq, out=(hb["block_table"][:n], hb["seq_lens"][:n], hb["slots"][:n]))
            ctx = hb["seq_lens"][:n]
            hb["positions"][:n] = ctx
            max_ctx = int(ctx.max()) + 1
            hb["seq_lens"][:n] += 1
        ids_np, keys_np, rem_np = hb["ids"].numpy(), hb["keys"].numpy(), hb["remaining"].numpy()
        for j, sid in enumerate(decode):
            r = reqs[sid]
            ids_np[j] = r.out_tokens[-1]
            keys_np[j] = self._row_key(r, sp)
            rem_np[j] = r.max_new - len(r.out_tokens)
        if self.hybrid:
            hb["state_rows"].zero_()    # padding rows use the scratch row
            for j, sid in enumerate(decode):
                hb["state_rows"][j] = self._state_row[sid]
        hb["active"][:n] = 1
        hb["win_step"][0] = 0
        B = self._bucket(max(n, 1))
        if B > n:  # padding rows: never active, no cache write, empty context
            for name in ("seq_lens", "ids", "positions", "keys", "active", "remaining"):
                hb[name][n:B] = 0
            hb["slots"][n:B] = -1
            hb["block_table"][n:B] = 0
        if steps is None:
            steps = self._window_steps(decode, reqs)
        if self.record_routing:
            steps = 1
            self._r3_rows(list(decode), hb["positions"][:n].clone()) if n else self._r3_rows([], [])
        st["blob"].copy_(st["host_blob"], non_blocking=True)   # all inputs of the window in one upload
        _L.Counters.h2d_bytes += st["host_blob"].numel()
        self._step_counter += steps
        self._run_decode(max(n, 1), sp, max_ctx, steps)
        if n == 0:
            self.stats["decode_s"] += time.perf_counter() - t0
            return
        both = _L.to_host(st["out_blob"])   # one download for the window; synchronises the stream
        if self._ev_pending:
            self.stats["decode_device_s"] += self._ev[0].elapsed_time(self._ev[1]) * 1e-3
            self._ev_pending = False
        Bm, W = self.max_running, self.decode_window
        prod = both[:n].tolist()
        toks = both[Bm : Bm + W * Bm].view(W, Bm)
        lps = both[Bm + W * Bm :].view(torch.float32).view(W, Bm)
        fin = [0] * n
        for j, sid in enumerate(decode):
            c = prod[j]
            if c <= 0:
                raise _L.NativeLibraryError(f"decode window produced no token for request {sid}")
            r = reqs[sid]
            r.out_tokens.extend(toks[:c, j].tolist())
            r.out_logprobs.extend(lps[:c, j].tolist())
            fin[j] = 1 if r.out_tokens[-1] in stop else 0
        fin = self.sched.commit_n(decode, prod, fin)
        for j, sid in enumerate(decode):
            if fin[j]:
                r = reqs[sid]
                r.finished = True
                r.truncated = fin[j] == 2 and r.out_tokens[-1] not in stop
                if self.finish_hook is not None:
                    self.finish_hook(r)
        self.stats["decode_steps"] += steps
        self.stats["generated_tokens"] += sum(prod)
        self.stats["decode_s"] += time.perf_counter() - t0

    # ------------------------------------------------------------------ public API
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams, max_new_tokens: Optional[Sequence[int]] = None,
                 share_prefixes: bool = True, request_uids: Optional[Sequence[int]] = None,
                 mm_inputs: Optional[Sequence] = None) -> list[_Request]:
        """Runs all prompts to completion with continuous batching. Returns one record per prompt (in input order)
        with the generated tokens, their log-probabilities and whether generation was cut by the length limit.
        ``mm_inputs``: per prompt ``(patches [n, patch_dim], [patches per image])`` or None, for vision-language models whose
        prompts hold one image placeholder token per patch row."""
        # inference keeps all rows on every tensor-parallel rank (all-reduce form), whatever the training layout is
        saved = self.tp.sequence_parallel if self.tp is not None else False
        if self.tp is not None:
            self.tp.sequence_parallel = False
        # no kernel of a generation phase writes a weight, so the decode GEMMs may start their weight stream early
        prev_static = E.skinny_static_weights(os.environ.get("RLB_SKINNY_EARLY_WEIGHTS", "1") != "0") if self.native else 0
        try:
            if self.quantization:
                from .quantized import quantized_inference

                with quantized_inference(True):
                    return self._generate(prompts, sp, max_new_tokens, share_prefixes, request_uids, mm_inputs)
            return self._generate(prompts, sp, max_new_tokens, share_prefixes, request_uids, mm_inputs)
        finally:
            if self.native:
                E.skinny_static_weights(bool(prev_static))
            if self.tp is not None:
                self.tp.sequence_parallel = saved

    @torch.no_grad()
    def _generate(self, prompts, sp: SamplingParams, max_new_tokens=None, share_prefixes: bool = True, request_uids=None,
                  mm_inputs=None) -> list[_Request]:
        self.wake()
        self.model.eval()
        stop = set(int(t) for t in (sp.stop_token_ids or []))
        reqs: dict[int, _Request] = {}
        first_of: dict[tuple, int] = {}
        for i, p in enumerate(prompts):
            p = [int(t) for t in p]
            mx = int(max_new_tokens[i]) if max_new_tokens is not None else sp.max_new_tokens
            mx = max(1, min(mx, self.max_model_len - len(p)))
            share = -1
            mm = mm_inputs[i] if mm_inputs is not None else None
            if mm is not None and mm[0] is None:
                mm = None
            if share_prefixes and not self.hybrid and not self.record_routing:   # (shared pages carry no state / no routing record)
                key = tuple(p)
                if mm is not None:   # equal prompts share their prefix only if they show the same images
                    from rl_b200.data.multimodal_utils import content_key

                    key = (key, content_key(mm[0]))
                if key in first_of:
                    share = first_of[key]
                else:
                    first_of[key] = i
            reqs[i] = _Request(i, p, mx, share_with=share, uid=int(request_uids[i]) if request_uids is not None else i)
            reqs[i].mm = mm
            if self.sched.add(i, len(p), mx, share) != 0:
                raise ValueError(f"request {i} (prompt {len(p)} + {mx} new tokens) can never fit the KV cache")
            if self.prefix_caching and mm is None and not self.record_routing:
                self.sched.set_hashes(i, self._block_hashes(p))
        dev = self.device
        st = self._static_buffers()
        if self.native and len(stop) > self.MAX_STOP_IDS:
            raise ValueError(f"at most {self.MAX_STOP_IDS} stop token ids are supported")
        self._n_stop = len(stop)
        st["host"]["stop_ids"].zero_()
        if stop and self.native:
            st["host"]["stop_ids"][: len(stop)] = torch.tensor(sorted(stop), dtype=torch.int32)
        t_begin = time.perf_counter()
        last_logits: dict[int, torch.Tensor] = {}
        # Expert-parallel MoE layers exchange tokens between the ranks of the expert group in every forward pass, so those
        # ranks must run the same sequence of forward passes although each serves its own requests: every iteration they
        # agree on whether a decode and / or a prefill pass happens, and a rank without work of that kind runs it on one
        # dummy token (no cache write, output discarded).
        ep = getattr(self.model, "ep", None)
        lock = ep is not None and ep.world > 1 and self.cfg.is_moe
        while True:
            if self.window_hook is not None:   # between two host visits (e.g. an in-flight weight update)
                self.window_hook()
            if self.admit_hook is not None and not lock:
                for p, mx, uid, tag in self.admit_hook():
                    rid = (max(reqs) + 1) if reqs else 0
                    p = [int(t) for t in p]
                    mx = max(1, min(int(mx) if mx is not None else sp.max_new_tokens, self.max_model_len - len(p)))
                    r = _Request(rid, p, mx, uid=int(uid))
                    r.tag = tag
                    if self.sched.add(rid, len(p), mx, -1) != 0:
                        r.finished, r.truncated, r.error = True, True, "the request can never fit the KV cache"
                        if self.finish_hook is not None:
                            self.finish_hook(r)
                        continue
                    reqs[rid] = r
                    if self.prefix_caching and not self.record_routing:
                        self.sched.set_hashes(rid, self._block_hashes(p))
            idle = self.sched.idle()
            if not lock and idle:
                break
            prefill, shared, decode, copies = self.sched.schedule() if not idle else ([], [], [], [])
            if self.collect_timeline:
                self.timeline.append((time.perf_counter() - t_begin, len(decode), len(prefill) + len(shared),
                                      sum(1 for r in reqs.values() if not r.finished)))
            if not idle and not prefill and not shared and not decode:
                raise RuntimeError("scheduler made no progress (KV cache too small for a single request)")
            if self.hybrid:
                self._claim_state_rows(set(prefill) | set(decode))
            agreed_steps = None
            if lock:
                # one exchange per iteration: does anyone still work, decode, prefill; the largest decode batch (every rank
                # pads to its bucket) and the smallest window any decoding rank can run
                want = self._window_steps(decode, reqs) if (decode and self.native) else 0
                v = self._agree_max(ep, [0 if idle else 1, len(decode), 1 if prefill else 0, -want if want else -(1 << 20)])
                if v[0] == 0:
                    break
                need_decode, need_prefill = v[1] > 0, v[2] > 0
                if need_decode and self.native:
                    self._agreed_bucket = 0
                    self._agreed_bucket = self._bucket(v[1])
                    agreed_steps = max(1, -v[3])
            else:
                need_decode, need_prefill = bool(decode), bool(prefill)
            if need_decode and not decode:
                if self.native:
                    self._decode_window_native([], reqs, sp, stop, st, agreed_steps)
                else:
                    self._dummy_forward(decode=True)
            if need_prefill and not prefill:
                self._dummy_forward(decode=False)
            # ---- decode the sequences that were already running
            if decode and self.native:
                self._decode_window_native(decode, reqs, sp, stop, st, agreed_steps)
            elif decode:
                t0 = time.perf_counter()
                n = len(decode)
                hb = st["host"]
                bt, ctx_t, sl = self.sched.tables(decode, self.max_blocks_per_seq)
                hb["block_table"][:n], hb["seq_lens"][:n], hb["slots"][:n] = bt, ctx_t, sl
                ctx = hb["seq_lens"][:n]
                hb["positions"][:n] = ctx
                max_ctx = int(ctx.max()) + 1
                hb["seq_lens"][:n] += 1
                ids_np, keys_np = hb["ids"].numpy(), hb["keys"].numpy()
                for j, sid in enumerate(decode):
                    r = reqs[sid]
                    ids_np[j] = r.out_tokens[-1]
                    keys_np[j] = self._row_key(r, sp)
                    if self.hybrid:
                        hb["state_rows"][j] = self._state_row[sid]
                st["blob"].copy_(st["host_blob"], non_blocking=True)
                self._step_counter += 1
                self._r3_rows(list(decode), hb["positions"][:n].clone())
                tok, lp = self._run_decode(n, sp, max_ctx)
                tok_h, lp_h = _L.to_host(tok).tolist(), _L.to_host(lp).tolist()
                fin = [1 if t in stop else 0 for t in tok_h]
                fin = self.sched.commit(decode, fin)
                for j, sid in enumerate(decode):
                    r = reqs[sid]
                    r.out_tokens.append(tok_h[j])
                    r.out_logprobs.append(lp_h[j])
                    if fin[j]:
                        r.finished = True
                        r.truncated = fin[j] == 2 and tok_h[j] not in stop
                        if self.finish_hook is not None:
                            self.finish_hook(r)
                self.stats["decode_steps"] += 1
                self.stats["generated_tokens"] += n
                self.stats["decode_s"] += time.perf_counter() - t0
            # ---- prefill newly admitted sequences (and recomputed ones)
            if prefill or shared:
                t0 = time.perf_counter()
                if prefill:
                    items = []
                    for sid in prefill:
                        r = reqs[sid]
                        cached = self.sched.cached_prefix(sid) if (self.prefix_caching and not self.record_routing) else 0
                        items.append((sid, r.prompt + r.out_tokens, cached))
                    has_mm = any(getattr(reqs[sid], "mm", None) is not None for sid in prefill)
                    cap = max(1, self.max_prefill_tokens)
                    if has_mm or (all(c == 0 for _, _, c in items) and all(len(seq) <= cap for _, seq, _ in items)):
                        logits = self._prefill_plain(items, reqs, dev)
                    else:
                        logits = self._prefill_with_prefix(items, dev, cap)
                    for sid, row in logits.items():
                        last_logits[sid] = row
                    if self.prefix_caching:
                        for sid in prefill:   # the prompt's full blocks can now serve later requests with the same prefix
                            self.sched.register_prefix(sid)
                if copies:
                    src = torch.tensor([a for a, _ in copies], dtype=torch.int32, device=dev)
                    dst = torch.tensor([b for _, b in copies], dtype=torch.int32, device=dev)
                    for li in self._attn_layers:
                        E.block_copy(self.k_cache[li], self.v_cache[li], src, dst)
                new = list(prefill) + list(shared)
                rows = torch.stack([last_logits[sid] if sid in last_logits else last_logits[reqs[sid].share_with] for sid in new])
                self._step_counter += 1
                keys_new = torch.tensor([self._row_key(reqs[sid], sp) for sid in new], dtype=torch.int64, device=dev)
                tok, lp = E.sample(rows.contiguous(), temperature=sp.temperature, top_k=sp.top_k or 0, top_p=sp.top_p,
                                   greedy=sp.greedy, seed=self.BASE_SEED, row_keys=keys_new)
                tok, lp = self._agree(tok, lp)
                tok_h, lp_h = _L.to_host(tok).tolist(), _L.to_host(lp).tolist()
                fin = [1 if t in stop else 0 for t in tok_h]
                fin = self.sched.commit(new, fin, first=True)
                for j, sid in enumerate(new):
                    r = reqs[sid]
                    r.out_tokens.append(tok_h[j])
                    r.out_logprobs.append(lp_h[j])
                    if fin[j]:
                        r.finished = True
                        r.truncated = fin[j] == 2 and tok_h[j] not in stop
                        if self.finish_hook is not None:
                            self.finish_hook(r)
                # logits of a prompt are kept while siblings that share it may still be admitted
                pending_partners = {reqs[s].share_with for s in reqs if not reqs[s].out_tokens and reqs[s].share_with >= 0}
                for sid in list(last_logits):
                    if sid not in pending_partners:
                        del last_logits[sid]
                self.stats["generated_tokens"] += len(new)
                self.stats["prefill_s"] += time.perf_counter() - t0
        if self.native:   # every token download above synchronised the stream
            _L.raise_on_status("GenerationEngine.generate", self.device)
        if self.record_routing:
            self._r3_assemble(reqs)
        return [reqs[i] for i in range(len(prompts))]
