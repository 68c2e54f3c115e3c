"""Driver-side policy: one object in the controller process that owns a worker group of :class:`PolicyWorker` ranks, shards
every batch over the data-parallel axis, dispatches the call to the workers and puts the answers back together. Role of
nemo_rl/models/policy/lm_policy.py (``Policy``: ``get_logprobs`` / ``get_reference_policy_logprobs`` / ``train`` / ``generate`` /
``prepare_for_*`` / ``save_checkpoint`` over a ``RayWorkerGroup`` with sharding annotations pipeline x data x context x tensor
parallel).

The SPMD entrypoints (``torchrun examples/run_grpo.py``) do not need it: there every rank is its own driver. This facade is
for a single controller that drives training from one process -- a notebook, a service, the single-controller loop -- with the
same worker code underneath. Bulk tensors between the workers (gradients, activations, weights) travel over their own NCCL /
gloo groups; the control plane carries the batches in and the results out.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.distributed.named_sharding import NamedSharding
from rl_b200.distributed.virtual_cluster import VirtualCluster
from rl_b200.distributed.worker_groups import WorkerBuilder, WorkerGroup

AXES = ("pipeline_parallel", "data_parallel", "context_parallel", "tensor_parallel")
_MODEL_AXES = ["pipeline_parallel", "context_parallel", "tensor_parallel"]


class PolicyWorkerProcess:
    """What runs inside each worker process: joins the group's process group, builds the :class:`PolicyWorker` (and, on
    first use, its generation engine) and forwards calls to it."""

    def __init__(self, policy_cfg: dict, model_cfg: Optional[dict] = None, init_optimizer: bool = True, init_reference_model: bool = True,
                 seed: int = 0, weights_path: Optional[str] = None, optimizer_path: Optional[str] = None, tokenizer_cfg: Optional[dict] = None,
                 backend: Optional[str] = None):
        from rl_b200.distributed.launch import init_distributed
        from rl_b200.models.config import ModelConfig
        from rl_b200.policy.worker import PolicyWorker

        self.rank, self.world, self.device = init_distributed(backend)
        tok = None
        if tokenizer_cfg:
            from rl_b200.algorithms.utils import get_tokenizer

            tok = get_tokenizer(tokenizer_cfg)
        mc = ModelConfig(**model_cfg) if model_cfg else None
        self.worker = PolicyWorker(policy_cfg, model_cfg=mc, device=self.device, init_optimizer=init_optimizer,
                                   init_reference_model=init_reference_model, tokenizer=tok, seed=seed, weights_path=weights_path)
        if weights_path and optimizer_path:
            self.worker.load_checkpoint(weights_path, optimizer_path)
        self.generation = None

    # ---- scoring / training
    def get_logprobs(self, data, micro_batch_size=None):
        return self.worker.get_logprobs(data, micro_batch_size).cpu()

    def get_reference_policy_logprobs(self, data, micro_batch_size=None):
        return self.worker.get_reference_policy_logprobs(data, micro_batch_size).cpu()

    def get_topk_logits(self, data, k, micro_batch_size=None):
        return self.worker.get_topk_logits(data, k, micro_batch_size).cpu()

    def score(self, data, micro_batch_size=None):
        return self.worker.score(data, micro_batch_size).cpu()

    def train(self, data, loss_fn, eval_mode=False, gbs=None, mbs=None):
        out = self.worker.train(data, loss_fn, eval_mode, gbs=gbs, mbs=mbs)
        return {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in out.items()}

    # ---- generation (colocated with training on the same GPU)
    def _gen(self):
        if self.generation is None:
            self.generation = self.worker.build_generation()
        return self.generation

    def prepare_for_generation(self):
        from rl_b200.algorithms.grpo import refit_policy_generation

        refit_policy_generation(self.worker, self._gen())
        return True

    def generate(self, data, greedy=False):
        return self._gen().generate(data, greedy=greedy).cpu()

    def finish_generation(self):
        return self._gen().finish_generation()

    # ---- modes, checkpoints, end of life
    def prepare_for_training(self):
        return self.worker.prepare_for_training()

    def prepare_for_lp_inference(self):
        return self.worker.prepare_for_lp_inference()

    def finish_training(self):
        return self.worker.finish_training()

    def save_checkpoint(self, weights_path, optimizer_path=None, tokenizer_path=None, **kw):
        return self.worker.save_checkpoint(weights_path, optimizer_path, tokenizer_path, **kw)

    def load_checkpoint(self, weights_path, optimizer_path=None):
        return self.worker.load_checkpoint(weights_path, optimizer_path)

    def layout(self):
        st = self.worker.pstate
        return dict(rank=self.rank, world=self.world, tp=st.tp, pp=st.pp, cp=st.cp, dp=st.dp, tp_rank=st.tp_rank, pp_rank=st.pp_rank,
                    cp_rank=st.cp_rank, dp_rank=st.dp_rank, device=str(self.device))

    def shutdown(self):
        from rl_b200.distributed.launch import shutdown_distributed

        self.worker.shutdown()
        shutdown_distributed()
        return True


class Policy:
    """The controller's handle on a group of policy workers. ``cluster`` supplies one bundle per rank; the parallel sizes
    come from the policy config (``policy.parallel`` or the ``dtensor_cfg`` / ``megatron_cfg`` keys)."""

    def __init__(self, cluster: VirtualCluster, config: dict, tokenizer_cfg: Optional[dict] = None, name_prefix: str = "lm_policy",
                 init_optimizer: bool = True, init_reference_model: bool = True, weights_path: Optional[str] = None,
                 optimizer_path: Optional[str] = None, model_cfg: Optional[dict] = None, seed: int = 0, backend: Optional[str] = None,
                 env_vars: Optional[dict] = None):
        from rl_b200.policy.worker import parallel_sizes

        ps = parallel_sizes(config)
        world = cluster.world_size()
        model_ranks = ps["tp"] * ps["pp"] * ps["cp"]
        if world % model_ranks:
            raise ValueError(f"{world} bundles cannot hold replicas of {model_ranks} ranks (tp {ps['tp']} x pp {ps['pp']} x cp {ps['cp']})")
        self.cfg = config
        self.dp = world // model_ranks
        self.sharding = NamedSharding.from_sizes(world, pipeline_parallel=ps["pp"], data_parallel=self.dp, context_parallel=ps["cp"],
                                                 tensor_parallel=ps["tp"])
        builder = WorkerBuilder("rl_b200.policy.lm_policy.PolicyWorkerProcess", config, model_cfg, init_optimizer, init_reference_model, seed,
                                weights_path, optimizer_path, tokenizer_cfg, backend)
        self.worker_group = WorkerGroup(cluster, builder, name=name_prefix, sharding_annotations=self.sharding,
                                        env_vars=dict(config.get("env_vars") or {}, **(env_vars or {})))

    # ------------------------------------------------------------------ dispatch helpers
    def _sharded(self, method: str, shards: list, **common) -> list:
        fut = self.worker_group.run_all_workers_sharded_data(method, in_sharded_axes=["data_parallel"], replicate_on_axes=_MODEL_AXES,
                                                             output_is_replicated=_MODEL_AXES, data=shards, common_kwargs=common)
        return self.worker_group.get_all_worker_results(fut)

    def _all(self, method: str, *args, **kwargs) -> list:
        return self.worker_group.get_all_worker_results(self.worker_group.run_all_workers_single_data(method, *args, **kwargs))

    def _split(self, data: BatchedDataDict, batch_size: Optional[int] = None) -> list[BatchedDataDict]:
        if data.size % self.dp:
            raise ValueError(f"a batch of {data.size} samples does not divide over {self.dp} data-parallel ranks")
        return list(data.shard_by_batch_size(self.dp, batch_size=batch_size))

    @staticmethod
    def _join(parts: list, pad: Optional[dict] = None) -> BatchedDataDict:
        return BatchedDataDict.from_batches(parts, pad_value_dict=pad)

    # ------------------------------------------------------------------ PolicyInterface
    def get_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return self._join(self._sharded("get_logprobs", self._split(data), micro_batch_size=micro_batch_size))

    def get_reference_policy_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return self._join(self._sharded("get_reference_policy_logprobs", self._split(data), micro_batch_size=micro_batch_size))

    def get_topk_logits(self, data: BatchedDataDict, k: int, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return self._join(self._sharded("get_topk_logits", self._split(data), k=k, micro_batch_size=micro_batch_size))

    def score(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return self._join(self._sharded("score", self._split(data), micro_batch_size=micro_batch_size))

    def train(self, data: BatchedDataDict, loss_fn, eval_mode: bool = False, gbs: Optional[int] = None, mbs: Optional[int] = None) -> dict[str, Any]:
        """Every data-parallel rank receives its part of EVERY global batch, so all ranks take the same optimizer steps. The
        loss and gradient norm are already reduced over the ranks; per-micro-batch metrics of all ranks are concatenated."""
        gbs = gbs or self.cfg["train_global_batch_size"]
        res = self._sharded("train", self._split(data, batch_size=gbs), loss_fn=loss_fn, eval_mode=eval_mode, gbs=gbs, mbs=mbs)
        out = dict(res[0])
        merged: dict[str, list] = {}
        for r in res:
            for k, v in (r.get("all_mb_metrics") or {}).items():
                merged.setdefault(k, []).extend(v)
        out["all_mb_metrics"] = merged
        out["train_tokens"] = sum(int(r.get("train_tokens", 0)) for r in res)
        out["total_flops"] = sum(float(r.get("total_flops", 0.0)) for r in res)
        return out

    # ------------------------------------------------------------------ GenerationInterface (colocated engines)
    def build_generation(self, gen_cfg: Optional[dict] = None) -> "PolicyGeneration":
        """The generation side as an object of its own, the shape the training loops take (``policy, generation``)."""
        return PolicyGeneration(self, gen_cfg or self.cfg.get("generation") or {})

    def prepare_for_generation(self) -> bool:
        return all(self._all("prepare_for_generation"))

    def generate(self, data: BatchedDataDict, greedy: bool = False) -> BatchedDataDict:
        pad_id = (self.cfg.get("generation") or {}).get("pad_token_id", 0) or 0
        parts = self._sharded("generate", self._split(data), greedy=greedy)
        return self._join(parts, pad={"output_ids": pad_id, "logprobs": 0.0})

    def finish_generation(self) -> bool:
        return all(self._all("finish_generation"))

    # ------------------------------------------------------------------ modes, checkpoints, end of life
    def prepare_for_training(self):
        self._all("prepare_for_training")

    def prepare_for_lp_inference(self):
        self._all("prepare_for_lp_inference")

    def finish_training(self):
        self._all("finish_training")

    def save_checkpoint(self, weights_path: str, optimizer_path: Optional[str] = None, tokenizer_path: Optional[str] = None, **kw) -> None:
        self._all("save_checkpoint", weights_path, optimizer_path, tokenizer_path, **kw)

    def load_checkpoint(self, weights_path: str, optimizer_path: Optional[str] = None) -> None:
        self._all("load_checkpoint", weights_path, optimizer_path)

    def layouts(self) -> list[dict]:
        return self._all("layout")

    def shutdown(self) -> bool:
        return self.worker_group.shutdown(cleanup_method="shutdown")

    def __del__(self):
        try:
            self.worker_group.shutdown(force=True)
        except Exception:
            pass


class PolicyGeneration:
    """Generation interface over the policy's workers: their engines share the GPUs (and, at matching layout, the weight
    buffers) with the trainer, so "refit" is part of :meth:`prepare_for_generation` inside every worker."""

    def __init__(self, policy: Policy, cfg: dict):
        self.policy, self.cfg = policy, dict(cfg)

    def prepare_for_generation(self, *a, **k) -> bool:
        return self.policy.prepare_for_generation()

    def generate(self, data: BatchedDataDict, greedy: bool = False) -> BatchedDataDict:
        return self.policy.generate(data, greedy=greedy)

    def finish_generation(self, *a, **k) -> bool:
        return self.policy.finish_generation()

    def shutdown(self) -> bool:
        return True


class TeacherWorkerGroup:
    """A frozen teacher on GPUs of its own (``on_policy_distillation.non_colocated_teachers``): a worker group sized by the
    teacher's ``num_nodes x gpus_per_node`` with its own tensor / pipeline / context parallel sizes, scoring only -- no
    optimizer, no reference copy, no engine. Answers like the in-process teacher of ``rl_b200/algorithms/opd.py`` does. Role of
    nemo_rl/models/policy/teacher_worker_group.py."""

    def __init__(self, tcfg, policy_config: dict, cluster: Optional[VirtualCluster] = None, model_cfg: Optional[dict] = None,
                 tokenizer_cfg: Optional[dict] = None, backend: Optional[str] = None):
        from rl_b200.distributed.virtual_cluster import visible_gpu_count

        self.alias, self.model_name, self.cfg = tcfg.alias, tcfg.model_name, tcfg
        cfg = {k: v for k, v in policy_config.items() if k not in ("optimizer", "scheduler", "generation", "lora_cfg", "draft", "quant_cfg")}
        cfg.update(model_name=tcfg.model_name, precision=tcfg.precision, logprob_batch_size=tcfg.micro_batch_size)
        cfg["parallel"] = dict(tensor_parallel_size=tcfg.tensor_model_parallel_size, pipeline_parallel_size=tcfg.pipeline_model_parallel_size,
                               context_parallel_size=tcfg.context_parallel_size, expert_parallel_size=tcfg.expert_model_parallel_size)
        cfg.update(tcfg.overrides)
        self._own_cluster = cluster is None
        self.cluster = cluster or VirtualCluster([tcfg.gpus_per_node] * tcfg.num_nodes, use_gpus=visible_gpu_count() > 0, name=f"teacher-{tcfg.alias}")
        self.policy = Policy(self.cluster, cfg, tokenizer_cfg=tokenizer_cfg, name_prefix=f"teacher_{tcfg.alias}", init_optimizer=False,
                             init_reference_model=False, weights_path=tcfg.model_name if model_cfg is None else None, model_cfg=model_cfg,
                             backend=backend)

    def get_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return BatchedDataDict(reference_logprobs=self.policy.get_logprobs(data, micro_batch_size)["logprobs"])

    def get_topk_logits(self, data: BatchedDataDict, k: int, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return self.policy.get_topk_logits(data, k, micro_batch_size)

    def shutdown(self) -> bool:
        ok = self.policy.shutdown()
        if self._own_cluster:
            self.cluster.shutdown()
        return ok


def create_teacher_worker_groups(master_config: dict, model_cfg: Optional[dict] = None, tokenizer_cfg: Optional[dict] = None,
                                 backend: Optional[str] = None) -> tuple[dict, dict]:
    """One :class:`TeacherWorkerGroup` per distinct teacher checkpoint of ``on_policy_distillation`` and the alias -> group map."""
    from rl_b200.algorithms import opd

    cfg = opd.opd_cfg(master_config)
    groups = {t.alias: TeacherWorkerGroup(t, master_config["policy"], None, model_cfg, tokenizer_cfg, backend) for t in opd.create_teacher_configs(cfg)}
    return groups, opd.alias_to_group_alias(cfg)
