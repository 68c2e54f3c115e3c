"""Generation facade: the token-in / token-out contract of the algorithms over the in-house engine.

``generate(data, greedy)`` takes right-padded ``input_ids`` [B, S] with ``input_lengths`` [B] and returns
``output_ids`` [B, S'] (prompt + response, right-padded), ``generation_lengths``, ``unpadded_sequence_lengths``,
``logprobs`` [B, S'] (zero on prompt and padding positions) and ``truncated`` — the shapes and meanings of
nemo_rl/models/generation/interfaces.py:291-380 and :392-527. Backends such as vLLM or SGLang are not wrapped: this
engine is the generation backend.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict

from .engine import GenerationEngine, SamplingParams

GENERATION_DEFAULTS = dict(
    backend="native",
    max_new_tokens=512,
    temperature=1.0,
    top_p=1.0,
    top_k=None,
    stop_token_ids=None,
    stop_strings=None,
    block_size=64,
    gpu_memory_utilization=0.5,
    kv_cache_tokens=None,
    max_model_len=None,
    max_running=512,
    max_prefill_tokens=16384,
    use_cuda_graphs=True,
    free_kv_cache_on_sleep=False,
    seed=0,
    precision="bfloat16",   # rollout precision of the linear layers: bfloat16 | mxfp8 | fp8 (vllm_cfg.precision in the reference)
)


def configure_generation_config(cfg: Optional[dict], tokenizer=None, is_eval: bool = False) -> dict:
    """Fills defaults: pad id and stop ids from the tokenizer's eos (the job of
    nemo_rl/models/generation/__init__.py:27-107)."""
    out = dict(GENERATION_DEFAULTS)
    out.update(cfg or {})
    if tokenizer is not None:
        out.setdefault("_pad_token_id", tokenizer.pad_token_id)
        if out.get("stop_token_ids") is None and getattr(tokenizer, "eos_token_id", None) is not None:
            out["stop_token_ids"] = [tokenizer.eos_token_id]
    out.setdefault("_pad_token_id", 0)
    return out


def verify_right_padding(data: BatchedDataDict, pad_value: int = 0) -> tuple[bool, str]:
    """Checks that every row of ``input_ids`` holds its tokens first and padding last."""
    ids = data["input_ids"]
    key = "input_lengths" if "input_lengths" in data else "unpadded_sequence_lengths"
    lens = data[key]
    B, S = ids.shape
    if (lens > S).any() or (lens < 0).any():
        return False, "lengths outside [0, S]"
    ar = torch.arange(S, device=ids.device)[None, :]
    pad_region = ar >= lens.to(ids.device)[:, None]
    if pad_region.any() and (ids[pad_region] != pad_value).any():
        return False, "non-pad token after the sequence end (left-padded input?)"
    return True, ""


class NativeGeneration:
    """Driver-facing generation object (one per GPU rank in the SPMD runtime)."""

    def __init__(self, model, cfg: Optional[dict] = None, tokenizer=None, pool_group=None, pool_stride: int = 1, split_group=None):
        """``pool_group``: the serving tensor-parallel group when it spans several data-parallel ranks of the trainer
        (each holding different prompts); the prompts of one rank per ``pool_stride`` consecutive ranks are pooled so that
        all ranks of the engine serve the same request set, and every rank gets its own results back."""
        self.pool_group, self.pool_stride = pool_group, max(1, int(pool_stride))
        # ``split_group``: ranks that hold the same prompts and complete serving weights (pipeline stages or context-parallel
        # ranks of one replica): each generates every S-th prompt and the results are exchanged
        self.split_group = split_group
        self.cfg = configure_generation_config(cfg, tokenizer)
        c = self.cfg
        self.tokenizer = tokenizer
        self.pad_id = int(c["_pad_token_id"] or 0)
        self.engine = GenerationEngine(
            model, block_size=c["block_size"], kv_cache_tokens=c["kv_cache_tokens"],
            gpu_memory_utilization=c["gpu_memory_utilization"], max_running=c["max_running"],
            max_prefill_tokens=c["max_prefill_tokens"], max_model_len=c["max_model_len"] or 8192,
            use_cuda_graphs=c["use_cuda_graphs"], tokenizer=tokenizer,
            quantization=(c.get("native_cfg") or {}).get("precision") or (c.get("vllm_cfg") or {}).get("precision") or c.get("precision"))
        self._calls = 0

    # lifecycle hooks of the generation contract
    def prepare_for_generation(self, *args, **kw) -> bool:
        self.engine.wake()
        self.last_quantization = self.engine.requantize()   # the weights may have moved since the last rollout
        return True

    def finish_generation(self, *args, **kw) -> bool:
        self.engine.sleep(free_kv_cache=bool(self.cfg["free_kv_cache_on_sleep"]))
        return True

    # ------------------------------------------------------------------ weights from a trainer outside this job
    def init_collective(self, rank_prefix: int, ip: str, port: int, world_size: int, *, train_world_size: int = 1) -> None:
        """Joins the trainer's weight communicator as rank ``train_world_size + rank_prefix`` (``GenerationInterface.init_collective``)."""
        from rl_b200.distributed.stateless_group import StatelessProcessGroup

        self._collective = StatelessProcessGroup(ip, port, int(train_world_size) + int(rank_prefix), world_size)

    def prepare_refit_info(self, state_dict_info: Optional[dict] = None) -> None:
        """Names, shapes and dtypes the trainer is going to send (checked against what arrives)."""
        self._refit_info = dict(state_dict_info or {})

    def update_weights_from_collective(self) -> bool:
        """Receives the buckets of ``PolicyWorker.broadcast_weights_for_collective`` and copies every tensor into this engine's
        (possibly tensor-parallel) parameters; the KV cache and the prefix cache of the old weights are dropped."""
        from rl_b200.models.hf_io import load_hf_tensors
        from rl_b200.refit.packed_broadcast import _numel, unpack

        g = self._collective
        info = getattr(self, "_refit_info", None) or {}
        dev = self.engine.device
        while True:
            meta = g.broadcast_obj(None, 0)
            if meta is None:
                break
            for n, shape, dt in meta:
                if n in info and (tuple(info[n][0]) != tuple(shape)):
                    raise ValueError(f"{n}: announced shape {tuple(info[n][0])}, received {tuple(shape)}")
            size = sum(-(-_numel(s) * torch.empty((), dtype=d).element_size() // 16) * 16 for _, s, d in meta)
            buf = torch.empty(size, dtype=torch.uint8, device=dev)
            g.broadcast_bulk(buf, 0)
            got = dict(unpack(buf, meta))
            load_hf_tensors(self.engine.model, got.get, strict=False)
        self.invalidate_kv_cache()
        if getattr(self.engine, "quantization", None):
            self.engine.requantize()
        return True

    def update_weights_via_ipc_zmq(self) -> bool:
        """Colocated: the engine already addresses the trainer's buffers (or its arena was filled by the re-shard kernel)."""
        return True

    def get_collective_sender_spec(self) -> dict:
        return {"sender_rank": 0, "transport": "packed buckets over a stateless process group"}

    @property
    def requires_kv_scale_sync(self) -> bool:
        return False      # no FP8 KV cache: no scales to carry

    @property
    def blocks_training(self) -> bool:
        return True       # colocated engines share the trainer's GPUs: generation and training alternate

    def invalidate_kv_cache(self) -> bool:
        self.engine.sched.reset()
        return True

    def shutdown(self) -> bool:
        self.engine.sleep(True)
        return True

    def _sampling(self, greedy: bool) -> SamplingParams:
        c = self.cfg
        self._calls += 1
        return SamplingParams(temperature=float(c["temperature"]), top_p=float(c["top_p"]), top_k=int(c["top_k"] or 0),
                              max_new_tokens=int(c["max_new_tokens"]), stop_token_ids=c["stop_token_ids"], greedy=greedy,
                              seed=int(c["seed"]) * 7919 + self._calls)

    def generate(self, data: BatchedDataDict, greedy: bool = False) -> BatchedDataDict:
        ids, lens = data["input_ids"], data["input_lengths"]
        B = ids.shape[0]
        lens_l = lens.tolist()
        ids_cpu = ids.cpu()
        prompts = [ids_cpu[i, : lens_l[i]].tolist() for i in range(B)]
        sp = self._sampling(greedy)
        uids = data["rng_ids"].tolist() if "rng_ids" in data else None
        mm = None
        if "pixel_patches" in data:
            mm = [(data["pixel_patches"][i], data["image_sizes"][i]) for i in range(B)]
            assert self.pool_group is None, "vision inputs with pooled serving groups are not supported"
        if self.pool_group is not None:
            import torch.distributed as dist

            S = dist.get_world_size(self.pool_group)
            me = dist.get_rank(self.pool_group)
            box = [None] * S
            dist.all_gather_object(box, (prompts, uids), group=self.pool_group)
            leaders = list(range(0, S, self.pool_stride))          # one rank per group of ranks holding the same data
            pooled, pooled_uids, start = [], [], {}
            for l in leaders:
                start[l] = len(pooled)
                pooled += box[l][0]
                # request ids must stay unique inside the pooled batch
                pooled_uids += box[l][1] if box[l][1] is not None else [(l << 24) | j for j in range(len(box[l][0]))]
            allrecs = self.engine.generate(pooled, sp, request_uids=pooled_uids)
            mine = (me // self.pool_stride) * self.pool_stride
            recs = allrecs[start[mine] : start[mine] + B]
        elif self.split_group is not None:
            import torch.distributed as dist

            S, me = dist.get_world_size(self.split_group), dist.get_rank(self.split_group)
            mine = list(range(me, B, S))
            part = self.engine.generate([prompts[i] for i in mine], sp, request_uids=[uids[i] if uids is not None else i for i in mine],
                                        mm_inputs=[mm[i] for i in mine] if mm is not None else None)
            box = [None] * S
            dist.all_gather_object(box, [(i, r.prompt, r.out_tokens, r.out_logprobs, r.truncated) for i, r in zip(mine, part)],
                                   group=self.split_group)
            from .engine import _Request

            recs = [None] * B
            for chunk in box:
                for i, prompt, toks, lps, trunc in chunk:
                    recs[i] = _Request(i, prompt, len(toks), out_tokens=toks, out_logprobs=lps, finished=True, truncated=trunc)
        else:
            recs = self.engine.generate(prompts, sp, request_uids=uids, mm_inputs=mm)
        stop_strings = data.get("stop_strings") or self.cfg.get("stop_strings")
        if stop_strings and self.tokenizer is not None:
            self._apply_stop_strings(recs, stop_strings)
        out_len = max(len(r.prompt) + len(r.out_tokens) for r in recs) if recs else 0
        out_ids = torch.full((B, out_len), self.pad_id, dtype=torch.long)
        logprobs = torch.zeros((B, out_len), dtype=torch.float32)
        gen_lens = torch.zeros(B, dtype=torch.long)
        tot_lens = torch.zeros(B, dtype=torch.long)
        trunc = torch.zeros(B, dtype=torch.bool)
        for i, r in enumerate(recs):
            P, G = len(r.prompt), len(r.out_tokens)
            out_ids[i, :P] = torch.tensor(r.prompt, dtype=torch.long)
            out_ids[i, P : P + G] = torch.tensor(r.out_tokens, dtype=torch.long)
            logprobs[i, P : P + G] = torch.tensor(r.out_logprobs, dtype=torch.float32)
            gen_lens[i], tot_lens[i], trunc[i] = G, P + G, r.truncated
        out = BatchedDataDict({"output_ids": out_ids, "generation_lengths": gen_lens,
                               "unpadded_sequence_lengths": tot_lens, "logprobs": logprobs, "truncated": trunc})
        traces = [getattr(r, "routed_experts", None) for r in recs]
        if traces and all(t is not None for t in traces):
            # rollout routing replay: expert ids per position and MoE layer, -1 where a position was never run (the last token)
            re = torch.full((B, out_len) + tuple(traces[0].shape[1:]), -1, dtype=torch.int16)
            for i, t in enumerate(traces):
                re[i, : t.shape[0]] = t
            out["routed_experts"] = re
        return out

    def _apply_stop_strings(self, recs, stop_strings) -> None:
        """Cuts each response at the first token whose decoded prefix contains a stop string."""
        per_sample = isinstance(stop_strings, list) and stop_strings and isinstance(stop_strings[0], (list, type(None)))
        for i, r in enumerate(recs):
            ss = stop_strings[i] if per_sample else stop_strings
            if not ss:
                continue
            text = ""
            for t in range(len(r.out_tokens)):
                text = self.tokenizer.decode(r.out_tokens[: t + 1])
                if any(s in text for s in ss):
                    r.out_tokens = r.out_tokens[: t + 1]
                    r.out_logprobs = r.out_logprobs[: t + 1]
                    r.truncated = False
                    break

    def stats(self) -> dict[str, Any]:
        return dict(self.engine.stats)

    def serve_http(self, host: str = "127.0.0.1", port: int = 0, model_name: str = "policy"):
        """Exposes this engine through the OpenAI-compatible front end (``generation.expose_http_server`` in the
        reference's vLLM config); external agents then roll out against the weights the trainer keeps refitting. The
        returned handle has ``base_url``, ``begin_weight_update`` / ``end_weight_update`` and ``stop``."""
        from .http_server import ServerHandle, create_app

        self._http = ServerHandle(create_app(self.engine, self.tokenizer, model_name=model_name,
                                             default_max_tokens=int(self.cfg["max_new_tokens"])), host, port).start()
        return self._http
