"""Policy worker: one process per GPU holding the policy model, its sharded optimizer, an optional reference copy and
(when colocated) the generation engine that shares the same weight buffers.

One class with a parallelism spec replaces the reference's three worker backends (DTensor V1/V2 and Megatron:
nemo_rl/models/policy/workers/dtensor_policy_worker_v2.py:401-683, megatron_policy_worker.py:749-1125). The public
methods keep the reference's worker API: ``train``, ``get_logprobs``, ``get_reference_policy_logprobs``,
``get_topk_logits``, ``score``, ``prepare_for_training`` / ``prepare_for_lp_inference``, ``save_checkpoint`` /
``load_checkpoint`` and the refit hooks. All batches are packed (padding never reaches a GEMM), so "sequence packing"
and "dynamic batching" only choose how samples are grouped into micro-batches.

Normalisation contract: losses are divided by the *global* number of valid tokens / sequences of the optimizer step
(all ranks, all micro-batches), gradients are summed over ranks, so no rank-count factor appears anywhere.
"""

from __future__ import annotations

import contextlib
import os
import time
from typing import Any, Optional

import torch
import torch.distributed as dist

from rl_b200.algorithms.loss.interfaces import LossInputType, LossType
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.models.config import ModelConfig, preset
from rl_b200.models.transformer import CausalLM, PackedBatch, build_model
from rl_b200.policy.optimizer import LRSchedule, ShardedAdamW, build_optimizer
from rl_b200.ops import lib as _L
from rl_b200.ops.functional import Fp8Training as _Fn_fp8
from rl_b200.ops.lib import to_device, to_host
from rl_b200.utils.flops import transformer_flops

POLICY_DEFAULTS = dict(
    model_name=None,
    train_global_batch_size=32,
    train_micro_batch_size=4,
    logprob_batch_size=8,
    generation_batch_size=32,
    max_total_sequence_length=4096,
    precision="bfloat16",
    activation_checkpointing=False,
    max_grad_norm=1.0,
    grad_dtype="float32",
    logprob_chunk_size=None,
    make_sequence_length_divisible_by=1,
    offload_optimizer_for_logprob=False,
)


def _dp_info(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def parallel_sizes(policy_cfg: dict, num_layers: Optional[int] = None) -> dict:
    """tp / pp / cp / ep sizes and the sequence-parallel flag from ``policy.parallel`` (or, for configs written for the
    reference, ``dtensor_cfg`` / ``megatron_cfg`` keys)."""
    par = dict(policy_cfg.get("parallel") or {})
    dt, mg = policy_cfg.get("dtensor_cfg") or {}, policy_cfg.get("megatron_cfg") or {}
    src = mg if mg.get("enabled") else dt

    def pick(k_new, *alts):
        if par.get(k_new) is not None:
            return par[k_new]
        for a in alts:
            if src.get(a) is not None:
                return src[a]
        return None

    tp = int(pick("tensor_parallel_size", "tensor_parallel_size", "tensor_model_parallel_size") or 1)
    pp = int(pick("pipeline_parallel_size", "pipeline_model_parallel_size") or 1)
    # interleaved schedule: chunks of layers per pipeline rank, given directly or as layers per chunk (Megatron's two spellings)
    vpp = int(pick("virtual_pipeline_stages", "virtual_pipeline_model_parallel_size") or 1)
    per_chunk = src.get("num_layers_per_virtual_pipeline_stage")
    if vpp <= 1 and per_chunk and num_layers:
        vpp = max(1, int(num_layers) // (pp * int(per_chunk)))
    if vpp > 1 and pp == 1:
        raise ValueError("virtual pipeline stages need pipeline_parallel_size > 1")
    return dict(tp=tp, pp=pp, vpp=max(1, vpp),
                cp=int(pick("context_parallel_size", "context_parallel_size") or 1),
                ep=int(pick("expert_parallel_size", "expert_model_parallel_size") or 1),
                sequence_parallel=bool(tp > 1 and (pick("sequence_parallel", "sequence_parallel") in (None, True))))


def _peak_tflops() -> float:
    """Dense bf16 peak of one GPU (what model-FLOPs utilisation is quoted against)."""
    from rl_b200.utils.flops import device_peak_tflops

    try:
        return float(device_peak_tflops(torch.cuda.get_device_name(0) if torch.cuda.is_available() else "B200"))
    except Exception:
        return float(device_peak_tflops("B200"))


def ensure_parallel(policy_cfg: dict):
    """Initialises the process-wide parallel layout from the policy config (idempotent; collective on first use)."""
    from rl_b200.parallel.state import get_state, init_parallel

    st = get_state()
    ps = parallel_sizes(policy_cfg)
    if st.world == 1 and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        st = init_parallel(ps["tp"], ps["pp"], ps["cp"], ps["ep"], ps["sequence_parallel"])
    return st


def _precision(name) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
            "float16": torch.float16}.get(str(name), torch.bfloat16)


class PolicyWorker:
    def __init__(self, policy_cfg: dict, model_cfg: Optional[ModelConfig] = None, device=None, dp_group=None,
                 init_optimizer: bool = True, init_reference_model: bool = True, tokenizer=None, seed: int = 0,
                 weights_path: Optional[str] = None, fused_comm=None):
        cfg = dict(POLICY_DEFAULTS)
        cfg.update(policy_cfg or {})
        self.cfg = cfg
        # rollout routing replay (``policy.router_replay.enabled``): the experts the engine chose for every position are forced
        # in the log-prob and training passes, so trainer and engine evaluate the same sub-network
        # (nemo_rl/models/megatron/train.py set_router_replay_forward)
        self.router_replay = bool((cfg.get("router_replay") or {}).get("enabled"))
        self.draft = self.draft_opt = None          # policy.draft / policy.quant_cfg: set up at the end of construction
        self.draft_loss_weight = 1.0
        self.quantizers: dict = {}
        st = ensure_parallel(cfg)
        self.pstate = st
        if st.world > 1 and st.tp * st.pp * st.cp > 1 and dp_group is None:
            # data parallel = the ranks that hold the same model shard; "self" when there is only one replica
            dp_group = st.dp_cp_group
            self.dp_group = None if dp_group == "self" else dp_group
            self.rank, self.world = (0, 1) if dp_group == "self" else (st.dp_rank * st.cp + st.cp_rank, st.dp * st.cp)
        else:
            self.dp_group = dp_group
            self.rank, self.world = _dp_info(dp_group)
        dp_group = self.dp_group
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.tokenizer = tokenizer
        dtype = _precision(cfg["precision"])
        name = cfg.get("model_name")
        overrides = cfg.get("hf_config_overrides") or {}
        if model_cfg is None:
            if name in (None, ""):
                raise ValueError("policy.model_name or an explicit ModelConfig is required")
            from rl_b200.models.config import PRESETS

            if name in PRESETS:
                model_cfg = preset(name, **overrides)
            elif os.path.isdir(name):
                model_cfg = ModelConfig.from_pretrained(name, **overrides)
                weights_path = weights_path or name
            else:
                raise ValueError(f"unknown model '{name}': give a preset name or a local HF checkpoint directory")
        self.model_cfg = model_cfg
        dtc = cfg.get("dtensor_cfg") or {}
        act_ckpt = bool(cfg.get("activation_checkpointing") or dtc.get("activation_checkpointing", False))
        from rl_b200.parallel.expert import EP
        from rl_b200.parallel.tensor import TP

        self.tp = TP.from_state(st)
        self.ep = EP.from_state(st)
        if self.tp.world > 1 and self.device.type == "cuda" and dtype == torch.bfloat16 and cfg.get("fused_tensor_parallel", True) \
                and st.tp_comm is None:
            try:
                from rl_b200.parallel.tensor import TPFusedComm

                st.tp_comm = TPFusedComm(st.tp_group, wait_limit_s=float(cfg.get("peer_wait_limit_s", 10.0)))
            except Exception as e:  # no peer access between these GPUs: NCCL collectives around the plain GEMM
                print(f"[policy] fused tensor-parallel kernels unavailable ({type(e).__name__}: {e}); using NCCL")
        self.tp.comm = st.tp_comm
        from rl_b200.parallel.context import CP

        self.cp = CP.from_state(st)
        lora = cfg.get("lora_cfg") or (cfg.get("dtensor_cfg") or {}).get("lora_cfg") or ((cfg.get("megatron_cfg") or {}).get("peft"))
        self.lora_cfg = dict(lora) if (lora and lora.get("enabled")) else None
        n_layers = model_cfg.num_hidden_layers if model_cfg is not None else None
        if n_layers is None and weights_path and os.path.exists(os.path.join(weights_path, "config.json")):
            import json

            with open(os.path.join(weights_path, "config.json")) as f:
                n_layers = json.load(f).get("num_hidden_layers")
        self.vpp = parallel_sizes(cfg, n_layers)["vpp"] if st.pp > 1 else 1
        mp = dict(tp=self.tp, ep=self.ep if self.ep.world > 1 else None, pp_rank=st.pp_rank, pp_size=st.pp, cp=self.cp, vpp=self.vpp)
        if weights_path:
            from rl_b200.models.hf_io import load_pretrained

            self.model = load_pretrained(weights_path, device=self.device, dtype=dtype, lora=self.lora_cfg, **mp)
            self.model.activation_checkpointing = act_ckpt
        else:
            self.model = build_model(model_cfg, device=self.device, dtype=dtype, seed=seed, activation_checkpointing=act_ckpt,
                                     lora=self.lora_cfg, **mp)
        # Hybrid sharding (HSDP; ``dtensor_cfg.dp_replicate_size`` / ``parallel.data_parallel_replicate_size`` = R): the
        # data-parallel ranks form R shard groups of dp / R consecutive ranks (a node each); optimizer state is cut inside a
        # shard group and gradient slices are all-reduced across the groups (nemo_rl/models/automodel/setup.py:464-509).
        par_h, dt_h = cfg.get("parallel") or {}, cfg.get("dtensor_cfg") or {}
        rep = int(par_h.get("data_parallel_replicate_size") or par_h.get("hsdp_replicas") or dt_h.get("dp_replicate_size") or dt_h.get("hsdp_replicas") or 1)
        self.shard_group, self.replicate_group = dp_group, None
        if rep > 1 and self.world > 1:
            if st.tp * st.pp * st.cp * st.ep > 1:
                raise NotImplementedError("hybrid sharding is available for plain data-parallel layouts")
            if self.world % rep:
                raise ValueError(f"dp_replicate_size {rep} must divide the data-parallel size {self.world}")
            ranks = dist.get_process_group_ranks(dp_group) if dp_group is not None else list(range(dist.get_world_size()))
            S = self.world // rep
            for r0 in range(0, self.world, S):          # collective: every rank creates every group, in the same order
                grp = dist.new_group(ranks=ranks[r0 : r0 + S]) if S > 1 else "self"
                if r0 <= self.rank < r0 + S:
                    self.shard_group = grp
            for j in range(S):
                grp = dist.new_group(ranks=ranks[j::S])
                if self.rank % S == j:
                    self.replicate_group = grp
        # On several GPUs of one node the flat parameter / gradient buffers live in peer-mapped memory so that the
        # optimizer step can run as one fused kernel over NVLink (rl_b200/csrc/comm.cu); NCCL is the fallback.
        model_parallel = st.tp * st.pp * st.cp * st.ep > 1 or self.replicate_group is not None
        if fused_comm is None and self.world > 1 and self.device.type == "cuda" and cfg.get("fused_optimizer", True) \
                and dtype == torch.bfloat16 and init_optimizer and not model_parallel and self.lora_cfg is None:
            try:
                from rl_b200.parallel.symmetric import FusedOptimizerComm

                fused_comm = FusedOptimizerComm(dp_group, wait_limit_s=float(cfg.get("peer_wait_limit_s", 20.0)))
            except Exception as e:  # no peer access between these GPUs: keep NCCL
                if self.rank == 0:
                    print(f"[policy] fused peer-memory optimizer unavailable ({type(e).__name__}: {e}); using NCCL")
                fused_comm = None
        # block-scaled FP8 training of the dense linear layers (policy.fp8_cfg / megatron_cfg.fp8_cfg, recipe mxfp8); the
        # embedding, output head, router and norms stay in bf16
        from rl_b200.ops import functional as _Fn

        fp8_cfg = cfg.get("fp8_cfg") or (cfg.get("megatron_cfg") or {}).get("fp8_cfg") or (cfg.get("dtensor_cfg") or {}).get("fp8_cfg")
        self.fp8_training = _Fn.Fp8Training.configure(fp8_cfg) if (fp8_cfg or _Fn.Fp8Training.enabled) else False
        if self.fp8_training:
            for n_, p_ in self.model.named_parameters():
                if n_.endswith(("embed_tokens", "lm_head", "score", "router")) or ".mlp.router" in n_ or p_.dim() != 2:
                    p_._rlb_keep_bf16 = True
        par_cfg = cfg.get("parallel") or {}
        self.full_sharding = (par_cfg.get("data_parallel_sharding") or dtc.get("data_parallel_sharding") or "optimizer") == "full"
        if self.full_sharding:
            if cfg.get("quant_cfg") or (cfg.get("draft") or {}).get("enabled"):
                raise NotImplementedError("quantisation-aware training and draft heads need resident parameters (data_parallel_sharding: optimizer)")
            return self._init_fully_sharded(cfg, st, dp_group, dtype, init_optimizer, init_reference_model)
        self.sharder = None
        self.fused_comm = fused_comm
        # expert-parallel MoE: expert weights differ between the ranks of an expert-parallel group, so they live in their
        # own flat buffer whose gradients are reduced (and optimizer state sharded) over the ranks holding the SAME experts
        split_experts = self.ep.world > 1 and model_cfg.is_moe
        if self.ep.world > 1 and model_cfg.is_moe and self.device.type == "cuda" and dtype == torch.bfloat16 \
                and cfg.get("fused_expert_parallel", True) and st.ep_comm is None:
            try:
                from rl_b200.parallel.expert import EPFusedComm

                sp_cfg = cfg.get("sequence_packing") or {}
                max_tok = max(int(sp_cfg.get("train_mb_tokens") or 0), int(sp_cfg.get("logprob_mb_tokens") or 0),
                              cfg["max_total_sequence_length"] * max(cfg["train_micro_batch_size"], cfg["logprob_batch_size"]), 16384)
                st.ep_comm = EPFusedComm(st.ep_group, model_cfg.hidden_size, (max_tok + 64) * model_cfg.num_experts_per_tok,
                                         model_cfg.num_experts // self.ep.world, wait_limit_s=float(cfg.get("peer_wait_limit_s", 10.0)))
            except Exception as e:
                print(f"[policy] fused expert-parallel dispatch unavailable ({type(e).__name__}: {e}); using NCCL all-to-all")
        self.ep.comm = st.ep_comm
        expert_names = self.model.expert_param_names() if split_experts else set()
        dense = (lambda n: n not in expert_names) if split_experts else None
        self.flat_base = None
        if self.lora_cfg is not None:
            # LoRA: the base weights are frozen (no gradient buffer, no optimizer state, and they double as the reference
            # policy with the adapters switched off); only the adapters are trained
            assert not split_experts, "LoRA with expert parallelism is not supported"
            self.flat_base = self.model.flatten_parameters(align=256, include=lambda n: not CausalLM.is_lora_param(n))
            for p_ in self.flat_base.params:
                p_.requires_grad_(False)
            dense = CausalLM.is_lora_param
        self.flat = self.model.flatten_parameters(align=256 * max(1, self.world),
                                                  allocator=fused_comm.alloc_params if (fused_comm is not None and self.lora_cfg is None) else None,
                                                  include=dense)
        self.flat_e = None
        e_group, e_world = None, 1
        if split_experts:
            e_group, e_world = st.extras.get("expert_dp_group"), int(st.extras.get("expert_dp_size", 1))
            self.flat_e = self.model.flatten_parameters(align=256 * max(1, e_world), include=expert_names.__contains__)
        self.ref_flat: Optional[torch.Tensor] = None
        self.ref_flat_e: Optional[torch.Tensor] = None
        self._has_reference = bool(init_reference_model)
        if init_reference_model and self.lora_cfg is None:
            # the reference policy stays resident in HBM as a second flat buffer (no CPU swap)
            self.ref_flat = self.flat.flat.clone()
            if self.flat_e is not None:
                self.ref_flat_e = self.flat_e.flat.clone()
        self.optimizer: Optional[ShardedAdamW] = None
        self.optimizer_e: Optional[ShardedAdamW] = None
        self.scheduler: Optional[LRSchedule] = None
        if init_optimizer:
            gdt = _precision(cfg.get("grad_dtype", "float32")) if dtype == torch.bfloat16 else torch.float32
            self.flat.attach_grad_buffer(gdt, allocator=fused_comm.alloc_grads if (fused_comm is not None and gdt == torch.float32) else None)
            self.optimizer = build_optimizer(self.flat, cfg, group=(self.shard_group if self.replicate_group is not None else dp_group)
                                             if self.world > 1 or st.world == 1 else "self", fused_comm=fused_comm,
                                             replicate_group=self.replicate_group)
            if self.flat_e is not None:
                self.flat_e.attach_grad_buffer(gdt)
                self.optimizer_e = build_optimizer(self.flat_e, cfg, group=e_group if (e_world > 1 and e_group != "self") else "self")
                # distinct experts live on the ranks of an expert-parallel group: their squared norms add up over it
                self.optimizer_e.set_model_parallel([], 1, [st.ep_group])
            self._configure_model_parallel_grads()
            self.scheduler = LRSchedule(self.optimizer, cfg.get("scheduler"))
        self.pipeline = None
        if st.pp > 1:
            from rl_b200.parallel.pipeline import PipelineRunner

            div = self.tp.world if (self.tp.world > 1 and self.tp.sequence_parallel) else 1
            self.pipeline = PipelineRunner(self.model, st.pp_group, st.pp_rank, st.pp, model_cfg.hidden_size, dtype, self.device,
                                           rows_of=lambda item: int(item[0].input_ids.numel()) // div, vpp=self.vpp)
        self.generation = None
        self.temperature = 1.0
        self.train_top_k, self.train_top_p = None, 1.0   # the sampler's filters, mirrored in the training log-probabilities
        gen_cfg = cfg.get("generation") or {}
        if gen_cfg:
            self.temperature = float(gen_cfg.get("temperature", 1.0) or 1.0)
            self.train_top_k = int(gen_cfg["top_k"]) if gen_cfg.get("top_k") else None
            self.train_top_p = float(gen_cfg.get("top_p") or 1.0)
        self.timers: dict[str, float] = {}
        if cfg.get("quant_cfg"):
            self._init_quantization(cfg)
        dcfg = cfg.get("draft") or {}
        if dcfg.get("enabled"):
            self._init_draft(dcfg, dtype, init_optimizer)

    # ------------------------------------------------------------------ quantisation-aware training
    def _init_quantization(self, cfg: dict) -> None:
        """``policy.quant_cfg`` (a built-in recipe name or a YAML recipe, see rl_b200/policy/qat.py): the chosen linear layers
        run through quantise-dequantise operators in training, scoring and generation. ``quant_calib_size`` > 0 calibrates the
        input ranges at start-up on ``quant_calib_data`` (a text / jsonl file; absent: random tokens) in batches of
        ``quant_batch_size`` sequences of ``quant_sequence_length`` tokens; without calibration input ranges are dynamic."""
        from rl_b200.policy import qat

        st = self.pstate
        if st.tp * st.pp * st.cp > 1 or getattr(self, "sharder", None) is not None:
            raise NotImplementedError("quantisation-aware training runs on data- / expert-parallel layouts with resident parameters")
        self.quant_recipe = qat.resolve_quant_cfg(str(cfg["quant_cfg"]))
        self.quantizers = qat.attach(self.model, self.quant_recipe)
        if not self.quantizers:
            raise ValueError(f"quant_cfg '{cfg['quant_cfg']}' enables no quantizer of this model")
        if int(cfg.get("quant_calib_size") or 0) > 0:
            self.calibrate_quantizers(None, int(cfg["quant_calib_size"]), int(cfg.get("quant_batch_size") or 8),
                                      int(cfg.get("quant_sequence_length") or min(512, cfg["max_total_sequence_length"])), cfg.get("quant_calib_data"))

    def calibrate_quantizers(self, data: Optional[BatchedDataDict] = None, num_samples: int = 64, batch_size: int = 8, seq_len: int = 512,
                             calib_file: Optional[str] = None) -> int:
        """Freezes the input quantizers' ranges from forward passes over ``data`` (or the file's texts, or random tokens)."""
        from rl_b200.policy import qat

        if data is None:
            V = self.model_cfg.vocab_size
            if calib_file and os.path.exists(calib_file) and self.tokenizer is not None:
                import json as _json

                rows = []
                with open(calib_file) as f:
                    for line in f:
                        line = line.strip()
                        if line:
                            try:
                                obj = _json.loads(line)
                                line = obj.get("text") or obj.get("article") or obj.get("prompt") or str(obj)
                            except ValueError:
                                pass
                            rows.append(self.tokenizer.encode(line)[:seq_len])
                        if len(rows) >= num_samples:
                            break
                lens = torch.tensor([max(1, len(r)) for r in rows])
                ids = torch.zeros((len(rows), int(lens.max())), dtype=torch.long)
                for i, r in enumerate(rows):
                    ids[i, : len(r)] = torch.tensor(r, dtype=torch.long)
            else:
                g = torch.Generator().manual_seed(1234 + self.rank)
                ids = torch.randint(0, V, (num_samples, seq_len), generator=g)
                lens = torch.full((num_samples,), seq_len)
            data = BatchedDataDict(input_ids=ids, input_lengths=lens)
        self.model.eval()

        def passes():
            for s0 in range(0, data.size, batch_size):
                mb = data.slice(s0, min(data.size, s0 + batch_size))
                yield lambda mb=mb: self._policy_logprobs(self._pack(mb)[0])

        n = qat.calibrate(self.quantizers, passes(), self.dp_group if self.world > 1 else None)
        self._weights_changed()
        return n

    def export_quantized(self, path: str) -> dict:
        """The deployment checkpoint of the quantised policy (packed 4-bit tensors, scales, ``hf_quant_config.json``)."""
        from rl_b200.policy import qat

        return qat.export_quantized(self.model, self.quantizers, path) if self.rank == 0 else {}

    # ------------------------------------------------------------------ draft head (speculative decoding)
    def _init_draft(self, dcfg: dict, dtype, init_optimizer: bool) -> None:
        """``policy.draft``: an EAGLE-3 style head trained beside the policy on the policy's own hidden states
        (``enabled``, ``model_name`` a directory to start from, ``loss_weight``, ``num_layers``, ``aux_layer_indices``,
        ``draft_vocab_size``). Role of nemo_rl/models/megatron/draft/utils.py::build_draft_model."""
        from rl_b200.models.draft import EagleDraft

        st = self.pstate
        if st.tp * st.pp * st.cp > 1 or getattr(self, "sharder", None) is not None:
            raise NotImplementedError("draft-head training runs on data-parallel layouts with resident parameters")
        self.draft = EagleDraft(self.model_cfg, dcfg.get("aux_layer_indices"), int(dcfg.get("num_layers") or 1), dcfg.get("draft_vocab_size"),
                                dtype=dtype, device=self.device)
        if dcfg.get("model_name"):
            self.draft.load_pretrained(str(dcfg["model_name"]))
        else:
            self.draft.init_head_from_policy(self.model.output_weight)
        self.draft_loss_weight = float(dcfg.get("loss_weight", 1.0))
        self.model.capture_layers = self.draft.aux_layers
        if init_optimizer:
            kw = dict((self.cfg.get("optimizer") or {}).get("kwargs") or {})
            self.draft_opt = torch.optim.AdamW(self.draft.parameters(), lr=float(kw.get("lr", 1e-5)), betas=tuple(kw.get("betas", (0.9, 0.999))),
                                               eps=float(kw.get("eps", 1e-8)), weight_decay=float(kw.get("weight_decay", 0.0)))

    def wrap_loss_with_draft(self, loss_fn):
        """The loss to hand to :meth:`train` when the draft head is trained along: policy loss + weight * draft loss."""
        if self.draft is None:
            return loss_fn
        from rl_b200.algorithms.loss.wrapper import DraftLossWrapper

        return DraftLossWrapper(loss_fn, draft_weight=self.draft_loss_weight)

    def _draft_inputs(self, batch: PackedBatch, S: int, mb: BatchedDataDict) -> dict:
        """Draft logits, their targets and mask for one micro-batch, from what the policy's forward left in ``captured``:
        position t reads the chosen hidden states at t and the embedding of token t + 1, and is scored against the policy's
        (detached, temperature-scaled) distribution at t + 1, i.e. over token t + 2."""
        from rl_b200.ops import functional as F

        cap = self.model.captured
        aux = torch.cat([cap[i].detach() for i in self.draft.aux_layers], dim=-1)
        nxt = torch.roll(cap["embeds"].detach(), -1, 0)        # (the last row of a sequence reads its neighbour's: masked below)
        d_logits = self.draft(aux, nxt, batch.positions, self.model.rope_freqs(), batch.cu_seqlens, batch.max_seqlen)
        with torch.no_grad():
            t_logits = F.linear(cap["final"].detach(), self.model.output_weight).float() / self.temperature
            t_logits = torch.roll(t_logits, -1, 0)
            if self.draft.draft_vocab != self.model_cfg.vocab_size:
                t_logits = t_logits.index_select(1, self.draft.target_ids())
        tm = mb["token_mask"].float()
        mask = torch.zeros_like(tm[:, 1:])
        mask[:, : max(0, tm.shape[1] - 2)] = tm[:, 2:]
        return dict(draft_logits=batch.unpack(d_logits, S)[:, :-1], target_logits=batch.unpack(t_logits, S)[:, :-1], draft_token_mask=mask)

    def _draft_step(self, max_norm: Optional[float]) -> float:
        params = [p for p in self.draft.parameters() if p.grad is not None]
        if self.world > 1:
            for p in params:
                dist.all_reduce(p.grad, group=self.dp_group)
        gn = torch.nn.utils.clip_grad_norm_(params, max_norm if max_norm else float("inf"))
        self.draft_opt.param_groups[0]["lr"] = self.optimizer.lr      # the draft follows the policy's schedule
        self.draft_opt.step()
        self.draft_opt.zero_grad(set_to_none=True)
        return float(gn)

    # ------------------------------------------------------------------ fully sharded parameters (ZeRO-3)
    def _init_fully_sharded(self, cfg, st, dp_group, dtype, init_optimizer: bool, init_reference_model: bool) -> None:
        """``parallel.data_parallel_sharding: full``: parameters, gradients and optimizer state are all sharded over the
        data-parallel ranks; units of the model are gathered on use (rl_b200/parallel/fsdp.py)."""
        from rl_b200.parallel.fsdp import ParamSharder, ShardOptimizer

        assert st.tp * st.pp * st.cp * st.ep == 1 and self.lora_cfg is None, "fully sharded parameters: data-parallel dense models"
        self.fused_comm = None
        self.sharder = ParamSharder(self.model, group=dp_group if self.world > 1 else "self",
                                    wait_limit_s=float(cfg.get("peer_wait_limit_s", 20.0)))
        self.model.sharder = self.sharder
        self.flat = self.flat_e = self.flat_base = None
        self.ref_flat = self.ref_flat_e = None
        self.ref_shard = self.sharder.p_shard.clone() if init_reference_model else None
        self._has_reference = bool(init_reference_model)
        self.optimizer = self.optimizer_e = self.scheduler = None
        if init_optimizer:
            spec = cfg.get("optimizer") or {}
            kw = dict(spec.get("kwargs") or {})
            self.optimizer = ShardOptimizer(self.sharder, lr=float(kw.get("lr", 1e-5)), betas=tuple(kw.get("betas", (0.9, 0.999))),
                                            eps=float(kw.get("eps", 1e-8)), weight_decay=float(kw.get("weight_decay", 0.01)),
                                            max_grad_norm=cfg.get("max_grad_norm"))
            self.scheduler = LRSchedule(self.optimizer, cfg.get("scheduler"))
        if self.world > 1:
            dist.barrier(group=dp_group)   # every shard is filled before anybody pulls from it
        self._replicated_runs = []
        self._tied_pp = False
        self.pipeline = None
        self.generation = None
        self.temperature = 1.0
        self.train_top_k, self.train_top_p = None, 1.0
        gen_cfg = cfg.get("generation") or {}
        if gen_cfg:
            self.temperature = float(gen_cfg.get("temperature", 1.0) or 1.0)
            self.train_top_k = int(gen_cfg["top_k"]) if gen_cfg.get("top_k") else None
            self.train_top_p = float(gen_cfg.get("top_p") or 1.0)
        self.timers = {}

    # ------------------------------------------------------------------ model-parallel gradient bookkeeping
    def _configure_model_parallel_grads(self) -> None:
        """Tells the optimizer which flat ranges are replicated over the tensor-parallel group (their squared norm counts
        once, and with sequence parallelism their gradients are partial sums that must be all-reduced) and over which
        groups the gradient norm has to be combined."""
        st = self.pstate
        self._replicated_runs: list[tuple[int, int]] = []
        if st.tp > 1:
            runs: list[list[int]] = []
            for n, o, k, _ in self.flat.named_slices():
                if self.model.is_tp_sharded(n):
                    continue
                end = o + -(-k // 8) * 8
                if runs and runs[-1][1] == o:
                    runs[-1][1] = end
                else:
                    runs.append([o, end])
            self._replicated_runs = [(a, min(b, self.flat.padded)) for a, b in runs]
        # tied embeddings under pipeline parallelism: the last stage holds a second copy of the table (for the output
        # projection); its gradient is all-reduced with the first stage's and its norm counted once
        self._tied_pp = bool(st.pp > 1 and self.model.embed_tokens is not None and self.model.lm_head is None
                             and not self.model_cfg.value_head and self.model_cfg.tie_word_embeddings)
        excluded = []
        if self._tied_pp and self.model.last_stage and not self.model.first_stage:
            for n, o, k, _ in self.flat.named_slices():
                if n == "embed_tokens":
                    excluded.append((o, o + k))
        if self.optimizer is not None:
            groups = [g for g in (st.tp_group if st.tp > 1 else None, st.pp_group if st.pp > 1 else None) if g is not None]
            self.optimizer.set_model_parallel(self._replicated_runs, st.tp, groups, excluded)

    def _sync_replicated_grads(self) -> None:
        """Sequence parallelism: every tp rank saw only its rows, so gradients of replicated parameters are partial."""
        st = self.pstate
        if self.flat is None or self.flat.grad is None:
            return
        if st.tp > 1 and st.sequence_parallel:
            self.flat.fold_autograd_grads()
            for a, b in self._replicated_runs:
                dist.all_reduce(self.flat.grad[a:b], group=st.tp_group)
        if getattr(self, "_tied_pp", False) and (self.model.first_stage or self.model.last_stage):
            self.flat.fold_autograd_grads()
            dist.all_reduce(self.model.embed_tokens.main_grad, group=st.extras["embed_group"])

    # ------------------------------------------------------------------ generation (colocated, shared weights)
    def build_generation(self, gen_cfg: Optional[dict] = None):
        """Creates the colocated generation engine over this worker's own weight buffers."""
        from rl_b200.engine.generation import NativeGeneration

        g = dict(self.cfg.get("generation") or {})
        g.update(gen_cfg or {})
        native_cfg = dict(g.get("native_cfg") or g.get("vllm_cfg") or {})
        merged = {k: v for k, v in g.items() if k not in ("native_cfg", "vllm_cfg", "colocated", "sglang_cfg")}
        for k in ("gpu_memory_utilization", "max_model_len", "block_size", "kv_cache_tokens", "max_running", "use_cuda_graphs"):
            if k in native_cfg:
                merged[k] = native_cfg[k]
        if native_cfg.get("enforce_eager"):
            merged["use_cuda_graphs"] = False
        merged.setdefault("max_model_len", self.cfg["max_total_sequence_length"])
        gen_tp = int(native_cfg.get("tensor_parallel_size") or self.tp.world)
        engine_model, pool_group, pool_stride, split_group = self.model, None, 1, None
        st = self.pstate
        if getattr(self, "sharder", None) is not None:
            # fully sharded trainer: the engine serves its own copy in the serving layout, rebuilt at every refit
            from rl_b200.parallel.fsdp import ShardedServingSync

            gen_tp = int(native_cfg.get("tensor_parallel_size") or 1)
            serve_group, comm, pool_group = self._serving_groups(gen_tp)
            self.weight_synchronizer = ShardedServingSync(self, gen_tp, serve_group, comm)
            engine_model, pool_stride = self.weight_synchronizer.serving_model, 1
        elif st.pp > 1:
            # every rank gets a serving copy of the whole model (the trainer's tensor-parallel layout), refreshed by packed
            # broadcasts over the pipeline group; the stages of one replica hold the same prompts and share the work
            from rl_b200.refit.packed_broadcast import PipelineWeightSynchronizer

            assert gen_tp == self.tp.world and st.ep == 1 and not self.model_cfg.is_moe, \
                "pipeline-parallel training serves with the trainer's tensor-parallel size (dense models)"
            self.weight_synchronizer = PipelineWeightSynchronizer(self.model, self.model_cfg, st)
            engine_model, split_group = self.weight_synchronizer.serving_model, st.pp_group
        elif gen_tp != self.tp.world:
            engine_model, pool_group, pool_stride, split_group = self._build_serving_layout(gen_tp)
        elif st.cp > 1:
            split_group = st.cp_group   # context-parallel ranks hold the same prompts and the same (full) weights
        self.generation = NativeGeneration(engine_model, merged, self.tokenizer, pool_group=pool_group, pool_stride=pool_stride,
                                           split_group=split_group)
        if self.router_replay and getattr(self.generation, "engine", None) is not None:
            self.generation.engine.set_record_routing(True)     # the engine files the experts it chose per position
        self.temperature = float(self.generation.cfg["temperature"] or 1.0)
        self.train_top_k = int(self.generation.cfg["top_k"]) if self.generation.cfg.get("top_k") else None
        self.train_top_p = float(self.generation.cfg.get("top_p") or 1.0)
        return self.generation

    def _serving_groups(self, gen_tp: int):
        """(serving tensor-parallel group, fused comm, pool group) for engines of ``gen_tp`` ranks cut from the job."""
        world = dist.get_world_size() if dist.is_initialized() else 1
        serve_group, comm = None, None
        if gen_tp > 1:
            assert world % gen_tp == 0, "generation tensor-parallel size must divide the world size"
            me = dist.get_rank()
            for g0 in range(0, world, gen_tp):  # collective: every rank creates every group
                grp = dist.new_group(ranks=list(range(g0, g0 + gen_tp)))
                if g0 <= me < g0 + gen_tp:
                    serve_group = grp
            if self.device.type == "cuda" and self.cfg.get("fused_tensor_parallel", True):
                try:
                    from rl_b200.parallel.tensor import TPFusedComm

                    comm = TPFusedComm(serve_group, wait_limit_s=float(self.cfg.get("peer_wait_limit_s", 10.0)))
                except Exception as e:
                    print(f"[policy] fused serving kernels unavailable ({type(e).__name__}: {e}); using NCCL")
        return serve_group, comm, (serve_group if gen_tp > 1 else None)

    def _build_serving_layout(self, gen_tp: int):
        """The engine serves with a tensor-parallel size different from the trainer's: every rank gets a weight arena in
        the serving layout, filled before each generation phase by the refit synchronizer (rl_b200/refit)."""
        from rl_b200.parallel.tensor import TPFusedComm
        from rl_b200.refit.synchronizer import WeightSynchronizer

        st = self.pstate
        assert st.pp * st.cp * st.ep == 1 and not self.model_cfg.is_moe and not self.model_cfg.is_hybrid, \
            "re-sharding refit covers dense tensor/data-parallel layouts of the attention + MLP families"
        world = dist.get_world_size() if dist.is_initialized() else 1
        assert world % gen_tp == 0, "generation tensor-parallel size must divide the world size"
        serve_group, comm = None, None
        if gen_tp > 1:
            me = dist.get_rank()
            for g0 in range(0, world, gen_tp):  # collective: every rank creates every group
                grp = dist.new_group(ranks=list(range(g0, g0 + gen_tp)))
                if g0 <= me < g0 + gen_tp:
                    serve_group = grp
            if self.device.type == "cuda" and self.cfg.get("fused_tensor_parallel", True):
                try:
                    comm = TPFusedComm(serve_group, wait_limit_s=float(self.cfg.get("peer_wait_limit_s", 10.0)))
                except Exception as e:
                    print(f"[policy] fused serving kernels unavailable ({type(e).__name__}: {e}); using NCCL")
        self.weight_synchronizer = WeightSynchronizer(self.model, self.model_cfg, gen_tp, group=None, serve_group=serve_group, serve_comm=comm)
        # ranks of one serving group that hold different data (more serving than training tensor parallelism) pool prompts
        pool = serve_group if gen_tp > self.tp.world else None
        # fewer serving than training tensor-parallel ranks: the tp / gen_tp engines inside one training group hold the
        # same prompts and complete weights, so they split the prompts (rank j of every engine forms one split group)
        split = None
        ttp = self.tp.world
        if gen_tp < ttp and world > 1:
            me = dist.get_rank()
            for g0 in range(0, world, ttp):   # collective: every rank creates every group
                for j in range(gen_tp):
                    grp = dist.new_group(ranks=[g0 + j + k * gen_tp for k in range(ttp // gen_tp)])
                    if g0 <= me < g0 + ttp and (me - g0) % gen_tp == j:
                        split = grp
        return self.weight_synchronizer.serving_model, pool, self.tp.world, split

    # ------------------------------------------------------------------ modes
    def prepare_for_training(self, *a, **k):
        self.model.train()
        for opt in (self.optimizer, self.optimizer_e):
            if opt is not None:
                opt.reload_state(self.device)

    def prepare_for_lp_inference(self, *a, **k):
        self.model.eval()
        if self.cfg.get("offload_optimizer_for_logprob"):
            for opt in (self.optimizer, self.optimizer_e):
                if opt is not None:
                    opt.offload_state()

    def finish_training(self, *a, **k):
        pass

    @contextlib.contextmanager
    def use_reference_weights(self):
        """Runs the model on the reference policy's weights by re-pointing every parameter at the second buffer (LoRA:
        by switching the adapters off)."""
        if self.lora_cfg is not None:
            self.model.set_adapters(False)
            try:
                yield
            finally:
                self.model.set_adapters(True)
            return
        if getattr(self, "sharder", None) is not None:
            assert self.ref_shard is not None, "the worker was built without a reference model"
            with self.sharder.use_shard(self.ref_shard):
                yield
            return
        assert self.ref_flat is not None, "the worker was built without a reference model"
        pairs = [(self.flat, self.ref_flat)] + ([(self.flat_e, self.ref_flat_e)] if self.flat_e is not None else [])
        try:
            for fl, ref in pairs:
                for p, o, n in zip(fl.params, fl.offsets, fl.numels):
                    p.data = ref[o : o + n].view(p.shape)
            self._weights_changed()
            yield
        finally:
            for fl, _ in pairs:
                for p, o, n in zip(fl.params, fl.offsets, fl.numels):
                    p.data = fl.flat[o : o + n].view(p.shape)
            self._weights_changed()

    # ------------------------------------------------------------------ weights to an engine outside this job
    def init_collective(self, ip: str, port: int, world_size: int, *, train_world_size: int = 1) -> None:
        """Joins a communicator that spans this trainer's rank 0 (as its rank 0) and the ranks of an external generation
        service (ranks 1..), outside both sides' default process groups (``PolicyInterface.init_collective`` of the reference).
        Ranks other than 0 of the trainer only take part in gathering their shards."""
        from rl_b200.distributed.stateless_group import StatelessProcessGroup

        self._collective = StatelessProcessGroup(ip, port, 0, world_size) if self.rank == 0 and self.pstate.rank == 0 else None

    def broadcast_weights_for_collective(self, kv_scales=None, bucket_bytes: int = 1 << 28) -> int:
        """Sends the current weights (HF names, gathered over tensor parallelism) to the generation ranks of
        :meth:`init_collective` in packed buckets: a small header through the group's store, the bytes through its bulk
        backend. Returns the payload bytes. The receiving side runs ``NativeGeneration.update_weights_from_collective``."""
        from rl_b200.models.hf_io import iter_hf_tensors
        from rl_b200.refit.packed_broadcast import _buckets, pack

        g = getattr(self, "_collective", None)
        total = 0
        for bucket in _buckets(((n, t.detach()) for n, t in iter_hf_tensors(self.model)), bucket_bytes):   # (collective over tp)
            if g is None:
                continue
            g.broadcast_obj([(n, tuple(t.shape), t.dtype) for n, t in bucket], 0)
            buf = pack([t for _, t in bucket], self.device)
            g.broadcast_bulk(buf, 0)
            total += buf.numel()
        if g is not None:
            g.broadcast_obj(None, 0)
        return total

    def stream_weights_via_ipc_zmq(self, *args, **kwargs) -> int:
        """Colocated engines read the trainer's own buffers (matching layouts) or are filled by the peer-memory re-shard kernel
        (``rl_b200/refit``): there is nothing to stream through host sockets. Kept so that callers written against the
        reference's colocated interface run; returns the bytes the synchronizer moved (0 for shared buffers)."""
        sync = getattr(self, "weight_synchronizer", None)
        if sync is not None:
            sync.sync_weights(None)
            return int(getattr(sync, "last_bytes", 0))
        return 0

    def offload_to_cpu(self) -> None:
        self.offload_before_refit()

    def _weights_changed(self) -> None:
        """Derived copies of the weights (quantised forms) are stale."""
        if getattr(self, "quantizers", None):
            from rl_b200.policy.qat import QatState

            QatState.weights_changed()

    # ------------------------------------------------------------------ micro-batching
    def _microbatches(self, data: BatchedDataDict, mbs: int, token_budget: Optional[int]):
        """Yields (micro-batch, original indices). With a token budget samples are bin-packed by length."""
        n = data.size
        if token_budget:
            from rl_b200.data.packing import get_packer

            algo = (self.cfg.get("sequence_packing") or {}).get("algorithm", "modified_first_fit_decreasing")
            lens = data["input_lengths"].tolist()
            cap = max(int(token_budget), max(lens) if lens else 1)
            for b in get_packer(algo, cap).pack(lens):
                yield data.select_indices(b), b
        else:
            for s in range(0, n, mbs):
                idx = list(range(s, min(n, s + mbs)))
                yield data.slice(s, min(n, s + mbs)), idx

    def _extra_passes(self, n_local: int) -> int:
        """Expert parallelism: every forward pass exchanges tokens inside the expert group, so its ranks must run the same
        number of passes although they hold different data. Returns how many dummy passes this rank has to add
        (the reference equalises micro-batch counts with zero-weight dummies as well: nemo_rl/models/automodel/data.py:201-254)."""
        if self.ep.world <= 1 or not self.model_cfg.is_moe:
            return 0
        t = torch.tensor([n_local], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.ep.group)
        return int(t.item()) - n_local

    def _dummy_pass(self, backward: bool) -> None:
        """One forward (+ backward) over a few padding tokens whose loss weight is zero."""
        ids = torch.zeros((1, 8), dtype=torch.long)
        batch, _ = self._pack(BatchedDataDict(input_ids=ids, input_lengths=torch.tensor([8])))
        with torch.set_grad_enabled(backward):
            lp, _ = self.model.next_token_logprobs(batch, self.temperature)
            if backward:
                (lp.sum() * 0.0).backward()

    def _policy_logprobs(self, batch: PackedBatch, h_in=None) -> torch.Tensor:
        """Per-token log-probabilities under the distribution the sampler draws from (temperature and, when the generation
        config uses them, top-k / top-p)."""
        if (self.train_top_k or 0) > 0 or self.train_top_p < 1.0:
            return self.model.next_token_logprobs_filtered(batch, self.train_top_k, self.train_top_p, self.temperature, h_in=h_in)
        return self.model.next_token_logprobs(batch, self.temperature, h_in=h_in)[0]

    def _token_budget(self, kind: str) -> Optional[int]:
        sp = self.cfg.get("sequence_packing") or {}
        db = self.cfg.get("dynamic_batching") or {}
        key = "train_mb_tokens" if kind == "train" else "logprob_mb_tokens"
        if sp.get("enabled"):
            return int(sp.get(key) or self.cfg["max_total_sequence_length"])
        if db.get("enabled"):
            return int(db.get(key) or self.cfg["max_total_sequence_length"])
        return None

    def _pack(self, mb: BatchedDataDict) -> tuple[PackedBatch, int]:
        ids = to_device(mb["input_ids"], self.device)
        lens = to_device(mb["input_lengths"], self.device)
        batch = PackedBatch.from_padded(ids, lens)
        if self.device.type == "cuda":
            batch.input_ids = batch.input_ids.to(torch.int32)
        if self.tp.world > 1 and self.tp.sequence_parallel:
            batch = batch.pad_to_multiple(8 * self.tp.world)
        elif self.cp.world > 1:
            batch = batch.pad_to_multiple(16 * self.cp.world)   # 2 cp chunks of whole 8-row groups
        if self.router_replay:
            self._set_router_replay(mb, lens, ids.shape[1], int(batch.input_ids.numel()))
        if "pixel_patches" in mb:   # vision-language batch: image patch rows in sample order (models/vision.py)
            parts = [t for t in mb["pixel_patches"] if t is not None]
            batch.mm = dict(patches=to_device(torch.cat(parts), self.device) if parts else None,
                            sizes=[int(x) for row in mb["image_sizes"] for x in (row or [])])
        return batch, ids.shape[1]

    def _set_router_replay(self, mb: BatchedDataDict, lens: torch.Tensor, S: int, packed_rows: int) -> None:
        """Hands every MoE layer the engine's expert choices for the rows of the next forward pass (packed order); without a
        record in the batch the routers decide themselves."""
        from rl_b200.utils import routing_trace as RT

        if self.pipeline is not None:
            raise NotImplementedError("rollout routing replay with pipeline parallelism")
        re = mb.get("routed_experts") if hasattr(mb, "get") else None
        if re is None:
            RT.replay(self.model, None)
            return
        re = to_device(re[:, :S], self.device)
        keep = torch.arange(S, device=self.device)[None, :] < lens[:, None].clamp(max=S)
        rows = re[keep]                                   # [T, MoE layers, k], the order PackedBatch.from_padded uses
        if rows.shape[0] < packed_rows:                   # rows appended for tensor / context parallel alignment
            rows = torch.cat([rows, rows.new_full((packed_rows - rows.shape[0],) + tuple(rows.shape[1:]), -1)])
        RT.replay_rows(self.model, rows)
        if os.environ.get("RLB_R3_TRACE"):      # the record as this pass sees it; `maybe_dump(model, ...)` after the pass writes the capture
            os.makedirs(os.environ["RLB_R3_TRACE"], exist_ok=True)
            self._r3_dumps = getattr(self, "_r3_dumps", 0) + 1
            torch.save(rows.cpu(), os.path.join(os.environ["RLB_R3_TRACE"], f"record_rank{self.rank}_{self._r3_dumps}.pt"))

    # ------------------------------------------------------------------ inference passes
    @torch.no_grad()
    def _logprob_pass(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> torch.Tensor:
        self.model.eval()
        n, S = data["input_ids"].shape
        out = torch.zeros((n, S), dtype=torch.float32)
        mbs = micro_batch_size or self.cfg["logprob_batch_size"]
        if self.pipeline is not None:
            items = [(*self._pack(mb), idx) for mb, idx in self._microbatches(data, mbs, self._token_budget("logprob"))]

            def stage(item, h_in):
                if self.model.at_output:
                    return self._policy_logprobs(item[0], h_in=h_in)
                return self.model.hidden_states(item[0], h_in)

            lps = self.pipeline.forward_only(items, stage, lambda item: (int(item[0].input_ids.numel()),))
            for (batch, Smb, idx), lp in zip(items, lps):
                out[torch.as_tensor(idx), :Smb] = to_host(batch.unpack(lp, Smb))
            return out
        mbl = list(self._microbatches(data, mbs, self._token_budget("logprob")))
        extra = self._extra_passes(len(mbl))  # agreed before the first pass: the count exchange is itself a collective
        for mb, idx in mbl:
            batch, Smb = self._pack(mb)
            lp = self._policy_logprobs(batch)
            out[torch.as_tensor(idx), :Smb] = to_host(batch.unpack(lp, Smb))
        for _ in range(extra):
            self._dummy_pass(backward=False)
        if self.device.type == "cuda":   # the downloads above synchronised the stream
            _L.raise_on_status("PolicyWorker log-probability pass", self.device)
        return out

    def get_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """{logprobs [B, S]}: log p(token t | tokens < t) under the current weights; position 0 is 0."""
        return BatchedDataDict({"logprobs": self._logprob_pass(data, micro_batch_size)})

    def get_reference_policy_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        with self.use_reference_weights():
            lp = self._logprob_pass(data, micro_batch_size)
        return BatchedDataDict({"reference_logprobs": lp})

    @torch.no_grad()
    def get_topk_logits(self, data: BatchedDataDict, k: int, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """Top-k next-token logits and their vocabulary ids for S-1 positions (teacher side of distillation)."""
        self.model.eval()
        n, S = data["input_ids"].shape
        vals = torch.zeros((n, S - 1, k), dtype=torch.float32)
        idxs = torch.zeros((n, S - 1, k), dtype=torch.long)
        mbs = micro_batch_size or self.cfg["logprob_batch_size"]
        for mb, idx in self._microbatches(data, mbs, None):
            batch, Smb = self._pack(mb)
            z = self.model.logits(batch) / self.temperature
            v, i = torch.topk(z, k, dim=-1)
            vals[torch.as_tensor(idx), : Smb - 1] = batch.unpack(v, Smb)[:, :-1].cpu()
            idxs[torch.as_tensor(idx), : Smb - 1] = batch.unpack(i, Smb)[:, :-1].cpu()
        return BatchedDataDict({"topk_logits": vals, "topk_indices": idxs})

    @torch.no_grad()
    def score(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """Reward-model / critic head: per-token values [B, S] and the value at each sequence's last token."""
        self.model.eval()
        n, S = data["input_ids"].shape
        vals = torch.zeros((n, S), dtype=torch.float32)
        mbs = micro_batch_size or self.cfg["logprob_batch_size"]
        for mb, idx in self._microbatches(data, mbs, None):
            batch, Smb = self._pack(mb)
            vals[torch.as_tensor(idx), :Smb] = batch.unpack(self.model.values(batch), Smb).cpu()
        last = (data["input_lengths"].long() - 1).clamp(min=0)
        return BatchedDataDict({"values": vals, "scores": vals.gather(1, last[:, None])[:, 0]})

    # ------------------------------------------------------------------ training
    def _loss_inputs(self, loss_fn, batch: PackedBatch, S: int, mb: BatchedDataDict, h_in=None) -> dict:
        """Model outputs in the form the loss wants. ``h_in``: the residual stream from the previous pipeline stage."""
        it = getattr(loss_fn, "input_type", LossInputType.LOGPROB)
        if it == LossInputType.LOGPROB:
            lp = self._policy_logprobs(batch, h_in=h_in)
            return {"next_token_logprobs": batch.unpack(lp, S)[:, 1:]}
        if it == LossInputType.VALUE:
            return {"values": batch.unpack(self.model.values(batch, h_in), S)}
        if it == LossInputType.LOGIT:
            if self.model_cfg.value_head:  # reward model: score at the last token of each sequence
                v = self.model.values(batch, h_in)
                ncu = batch.cu_seqlens[:-1] if batch.num_real_tokens is not None else batch.cu_seqlens
                last = (ncu[1:].long() - 1).clamp(min=0)
                return {"logits": v[last]}
            return {"logits": batch.unpack(self.model.logits(batch, h_in), S)}
        if it == LossInputType.DISTILLATION:
            z = self.model.logits(batch, h_in) / self.temperature
            logp = torch.log_softmax(batch.unpack(z, S)[:, :-1], dim=-1)
            ti = mb["teacher_topk_indices"].to(self.device)
            s_topk = logp[:, : ti.shape[1]].gather(-1, ti)
            t_topk = torch.log_softmax(mb["teacher_topk_logits"].to(self.device).float(), dim=-1)
            return {"student_topk_logprobs": s_topk, "teacher_topk_logprobs": t_topk}
        raise ValueError(f"unsupported loss input type {it}")

    def train(self, data: BatchedDataDict, loss_fn, eval_mode: bool = False, *, gbs: Optional[int] = None,
              mbs: Optional[int] = None) -> dict[str, Any]:
        """Runs optimizer steps over this rank's shard of ``data`` (``gbs`` counts samples over all ranks; each rank
        holds ``gbs / dp`` samples of every global batch). Returns loss / grad-norm / per-micro-batch metrics."""
        assert self.optimizer is not None or eval_mode
        if self.draft is not None and not getattr(loss_fn, "needs_draft_logits", False) \
                and getattr(loss_fn, "input_type", LossInputType.LOGPROB) == LossInputType.LOGPROB:
            loss_fn = self.wrap_loss_with_draft(loss_fn)      # every algorithm trains the draft head along with the policy
        gbs = gbs or self.cfg["train_global_batch_size"]
        mbs = mbs or self.cfg["train_micro_batch_size"]
        cpw = self.cp.world  # context-parallel ranks of one replica see the same samples
        local_gbs = max(1, gbs // max(1, self.world // cpw))
        n_local = data.size
        num_gb = max(1, n_local // local_gbs)
        self.model.train(not eval_mode)
        losses, grad_norms, all_mb_metrics = [], [], []
        total_tokens = 0
        t_start = time.perf_counter()
        for g in range(num_gb):
            gb = data.slice(g * local_gbs, min(n_local, (g + 1) * local_gbs))
            tm = gb["token_mask"][:, 1:].float() if "token_mask" in gb else None
            sm = gb["sample_mask"].float() if "sample_mask" in gb else torch.ones(gb.size)
            counts = torch.stack([sm.sum(), (tm * sm[:, None]).sum() if tm is not None else sm.sum()]).to(self.device)
            if self.world > 1:
                dist.all_reduce(counts, group=self.dp_group)
                counts = counts / cpw
            global_valid_seqs, global_valid_toks = counts[0], counts[1]
            if not eval_mode:
                self.optimizer.zero_grad()
                if self.optimizer_e is not None:
                    self.optimizer_e.zero_grad()
            gb_loss = torch.zeros((), device=self.device)
            budget = None if getattr(loss_fn, "requires_pairs", False) else self._token_budget("train")
            if self.pipeline is not None:
                gb_loss, mbm, ntok = self._pipeline_global_batch(gb, mbs, budget, loss_fn, eval_mode, global_valid_seqs, global_valid_toks)
                all_mb_metrics.extend(mbm)
                total_tokens += ntok
            mbl = list(self._microbatches(gb, mbs, budget)) if self.pipeline is None else []
            for _ in range(self._extra_passes(len(mbl)) if self.pipeline is None else 0):
                self._dummy_pass(backward=not eval_mode)
            for mb, _ in mbl:
                batch, S = self._pack(mb)
                mb_dev = BatchedDataDict({k: (to_device(v, self.device) if isinstance(v, torch.Tensor) else v)
                                          for k, v in mb.items() if k != "input_ids"})
                mb_dev.truncate_tensors(1, S)
                total_tokens += int(batch.input_ids.numel())
                with torch.set_grad_enabled(not eval_mode):
                    inputs = self._loss_inputs(loss_fn, batch, S, mb_dev)
                    if self.draft is not None and getattr(loss_fn, "needs_draft_logits", False):
                        inputs.update(self._draft_inputs(batch, S, mb_dev))
                    loss, metrics = loss_fn(data=mb_dev, global_valid_seqs=global_valid_seqs,
                                            global_valid_toks=global_valid_toks, **inputs)
                    if not eval_mode:
                        loss.backward()
                gb_loss += loss.detach()
                metrics = dict(metrics)
                metrics["lr"] = self.optimizer.lr if self.optimizer else 0.0
                metrics["global_valid_seqs"] = float(global_valid_seqs)
                metrics["global_valid_toks"] = float(global_valid_toks)
                all_mb_metrics.append(metrics)
            if not eval_mode:
                self._sync_replicated_grads()
                if self.optimizer_e is None:
                    gn = self.optimizer.step()
                else:  # dense and expert parameters share one clipping coefficient
                    total = self.optimizer.reduce_and_sumsq() + self.optimizer_e.reduce_and_sumsq()
                    gn = self.optimizer.apply(total.clone())
                    self.optimizer_e.lr = self.optimizer.lr
                    self.optimizer_e.apply(total.clone())
                grad_norms.append(gn)
                if self.draft_opt is not None and any(p.grad is not None for p in self.draft.parameters()):
                    draft_gn = self._draft_step(self.cfg.get("max_grad_norm"))
                    if all_mb_metrics:
                        all_mb_metrics[-1]["draft_grad_norm"] = draft_gn
                self._weights_changed()
                if getattr(self, "fp8_training", False):
                    _Fn_fp8.weights_changed()   # cached MXFP8 copies of the weights are stale now
            if self.world > 1:
                dist.all_reduce(gb_loss, group=self.dp_group)
                gb_loss = gb_loss / cpw
            losses.append(gb_loss)
        if not eval_mode and self.scheduler is not None:
            self.scheduler.step()  # once per train() call
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            _L.raise_on_status("PolicyWorker.train", self.device)   # a kernel that gave up a wait left garbage behind
        elapsed = time.perf_counter() - t_start
        mb_metrics: dict[str, list] = {}
        for m in all_mb_metrics:
            for k, v in m.items():
                mb_metrics.setdefault(k, []).append(v)
        flops = transformer_flops(self.model_cfg, total_tokens, self.cfg["max_total_sequence_length"], backward=not eval_mode)
        return {
            "loss": torch.stack(losses).cpu() if losses else torch.zeros(0),
            "grad_norm": torch.stack([g.reshape(()) for g in grad_norms]).cpu() if grad_norms else torch.zeros(0),
            "all_mb_metrics": mb_metrics,
            "total_flops": flops,
            "num_ranks": self.world,
            "theoretical_tflops": _peak_tflops(),
            "train_time_s": elapsed,
            "train_tokens": total_tokens,
        }

    def _pipeline_global_batch(self, gb, mbs, budget, loss_fn, eval_mode, global_valid_seqs, global_valid_toks):
        """One accumulation window through the pipeline schedule. Losses and metrics live on the last stage and are
        shared with the other stages afterwards so that every rank reports the same numbers."""
        items, ntok = [], 0
        for mb, _ in self._microbatches(gb, mbs, budget):
            batch, S = self._pack(mb)
            mb_dev = BatchedDataDict({k: (to_device(v, self.device) if isinstance(v, torch.Tensor) else v)
                                      for k, v in mb.items() if k != "input_ids"})
            mb_dev.truncate_tensors(1, S)
            items.append((batch, S, mb_dev))
            ntok += int(batch.input_ids.numel())
        collected: list[dict] = []

        def stage(item, h_in):
            batch, S, mb_dev = item
            if not self.model.at_output:
                return self.model.hidden_states(batch, h_in)
            inputs = self._loss_inputs(loss_fn, batch, S, mb_dev, h_in)
            loss, metrics = loss_fn(data=mb_dev, global_valid_seqs=global_valid_seqs, global_valid_toks=global_valid_toks, **inputs)
            collected.append(dict(metrics))
            return loss

        if eval_mode:
            with torch.no_grad():
                outs = self.pipeline.forward_only(items, stage, lambda item: (), torch.float32)
            losses = outs
        else:
            losses = self.pipeline.train_step(items, stage)
        st = self.pstate
        box = [collected, [float(x) for x in losses]] if self.model.last_stage else [None, None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(st.pp_group, st.pp - 1), group=st.pp_group)
        collected, loss_vals = box
        mbm = []
        for m in collected:
            m = dict(m)
            m["lr"] = self.optimizer.lr if self.optimizer else 0.0
            m["global_valid_seqs"] = float(global_valid_seqs)
            m["global_valid_toks"] = float(global_valid_toks)
            mbm.append(m)
        return torch.tensor(sum(loss_vals), device=self.device, dtype=torch.float32), mbm, ntok

    # ------------------------------------------------------------------ refit hooks
    def prepare_refit_info(self) -> dict:
        """name -> (shape, dtype) of every logical HF tensor (the refit wire format)."""
        from rl_b200.models.hf_io import iter_hf_tensors

        return {n: (tuple(t.shape), t.dtype) for n, t in iter_hf_tensors(self.model)}

    def offload_before_refit(self):
        pass

    def offload_after_refit(self):
        pass

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, weights_path: str, optimizer_path: Optional[str] = None, tokenizer_path: Optional[str] = None,
                        model_save_format: str = "safetensors", **kw) -> None:
        from rl_b200.checkpoint.io import save_optimizer_shard, save_weights

        save_weights(self, weights_path, model_save_format)
        if optimizer_path and self.optimizer is not None:
            save_optimizer_shard(self, optimizer_path, model_save_format)
        if tokenizer_path and self.tokenizer is not None and self.rank == 0:
            if hasattr(self.tokenizer, "save_pretrained"):
                self.tokenizer.save_pretrained(tokenizer_path)
            else:      # the built-in byte-level tokenizers have no files: record which one it was
                import json as _json

                os.makedirs(tokenizer_path, exist_ok=True)
                with open(os.path.join(tokenizer_path, "tokenizer_config.json"), "w") as f:
                    _json.dump({"tokenizer_class": type(self.tokenizer).__name__, "name": getattr(self.tokenizer, "name_or_path", None),
                                "vocab_size": len(self.tokenizer)}, f)
        if self.quantizers and self.rank == 0:      # calibrated input ranges travel with the weights
            from rl_b200.policy import qat

            torch.save(qat.state_dict(self.quantizers), os.path.join(os.path.dirname(os.path.abspath(weights_path)), "quantizers.pt"))
        if self.draft is not None and self.rank == 0:      # the draft head, in the EAGLE-3 checkpoint layout, beside the weights
            self.draft.save_pretrained(os.path.join(os.path.dirname(os.path.abspath(weights_path)), "draft"))
        if self.world > 1:
            dist.barrier(group=self.dp_group)

    def load_checkpoint(self, weights_path: str, optimizer_path: Optional[str] = None) -> None:
        from rl_b200.checkpoint.io import load_optimizer_shard, load_weights

        load_weights(self, weights_path)
        if optimizer_path and self.optimizer is not None and os.path.exists(optimizer_path):
            load_optimizer_shard(self, optimizer_path)
        self._weights_changed()
        qpath = os.path.join(os.path.dirname(os.path.abspath(weights_path)), "quantizers.pt")
        if self.quantizers and os.path.exists(qpath):
            from rl_b200.policy import qat

            qat.load_state_dict(self.quantizers, torch.load(qpath))
            for q in self.quantizers.values():
                if q.input_amax is not None:
                    q.input_amax = q.input_amax.to(self.device)
        dpath = os.path.join(os.path.dirname(os.path.abspath(weights_path)), "draft")
        if self.draft is not None and os.path.exists(os.path.join(dpath, "model.safetensors")):
            self.draft.load_pretrained(dpath)

    def shutdown(self) -> bool:
        if self.generation is not None:
            self.generation.shutdown()
        return True
