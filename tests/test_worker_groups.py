"""Virtual cluster and worker groups: placement, the three dispatch forms, result selection, failures, rendezvous of the
workers' own process group, and the driver-side policy facade on top of them."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.distributed.named_sharding import NamedSharding  # noqa: E402
from rl_b200.distributed.virtual_cluster import ResourceInsufficientError, VirtualCluster  # noqa: E402
from rl_b200.distributed.worker_groups import MultiWorkerFuture, WorkerBuilder, WorkerError, WorkerGroup  # noqa: E402


class EchoWorker:
    def __init__(self, tag, fail_on_rank=None):
        self.tag, self.rank, self.world = tag, int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        self.log = []
        if fail_on_rank is not None and self.rank == fail_on_rank:
            raise RuntimeError("cannot build")

    def whoami(self):
        return dict(rank=self.rank, world=self.world, tag=self.tag, local=int(os.environ["LOCAL_RANK"]), group=os.environ["RLB_WORKER_GROUP"])

    def add(self, x, y=0):
        self.log.append(("add", x, y))
        return None if x is None else x + y + self.rank * 1000

    def history(self):
        return list(self.log)

    def boom(self):
        raise ValueError(f"bad input on rank {self.rank}")

    def all_reduce_rank(self):
        import torch.distributed as dist

        if not dist.is_initialized():
            dist.init_process_group("gloo", rank=self.rank, world_size=self.world)
        t = torch.tensor([float(self.rank + 1)])
        dist.all_reduce(t)
        return float(t)

    def cleanup(self):
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
        open(os.environ["RLB_TEST_MARK"] + f".{self.rank}", "w").write("bye")


def test_virtual_cluster_shapes_and_limits():
    c = VirtualCluster([4, 4], use_gpus=False, max_colocated_worker_groups=2, name="c", node_addresses=["10.0.0.1", "10.0.0.2"])
    assert c.world_size() == 8 and c.node_count() == 2 and [b.node for b in c.bundles()] == [0] * 4 + [1] * 4
    assert c.claim_group() == 0 and c.claim_group() == 1
    with pytest.raises(ResourceInsufficientError):
        c.claim_group()
    c.release_group()
    a, b = c.split(6)
    assert a.world_size() == 6 and b.world_size() == 2 and b.node_addresses == ["10.0.0.2"] and a.bundle_ct_per_node_list == [4, 2]
    with pytest.raises(ResourceInsufficientError):
        VirtualCluster([9], use_gpus=True, num_gpus_per_node=8)
    with pytest.raises(ValueError):
        VirtualCluster([0])
    g = VirtualCluster([2], use_gpus=False)
    assert g.get_master_address_and_port()[0] == "127.0.0.1" and g.get_master_address_and_port()[1] > 0


def test_placement_prefers_few_nvlink_domains():
    from rl_b200.distributed.virtual_cluster import NodeInfo, cluster_from_nodes, place_on_nodes

    nodes = [NodeInfo("n1", 8, "rackA"), NodeInfo("n2", 8, "rackB"), NodeInfo("n3", 8, "rackA"), NodeInfo("n4", 4, "rackA"), NodeInfo("n5", 8, "rackB"),
             NodeInfo("n6", 8, "rackB"), NodeInfo("n7", 8, None)]
    assert [n.address for n in place_on_nodes(nodes, 2, 8)] == ["n1", "n3"]                 # the smallest domain that holds the job
    assert [n.address for n in place_on_nodes(nodes, 3, 8)] == ["n2", "n5", "n6"]           # only rack B holds three
    assert [n.address for n in place_on_nodes(nodes, 5, 8)] == ["n2", "n5", "n6", "n1", "n3"]     # largest domains first, kept together
    assert [n.address for n in place_on_nodes(nodes, 3, 4)][:3] == ["n1", "n3", "n4"]       # the 4-GPU node qualifies for 4-GPU bundles
    with pytest.raises(ResourceInsufficientError):
        place_on_nodes(nodes, 7, 8)
    c = cluster_from_nodes(nodes, 2, 8, use_gpus=False, name="t")
    assert c.node_addresses == ["n1", "n3"] and c.world_size() == 16


def test_worker_group_dispatch_forms_and_failures(tmp_path):
    cluster = VirtualCluster([4], use_gpus=False, name="t")
    sa = NamedSharding.from_sizes(4, data_parallel=2, tensor_parallel=2)
    mark = str(tmp_path / "mark")
    g = WorkerGroup(cluster, WorkerBuilder(EchoWorker, "hello"), name="echo", sharding_annotations=sa, env_vars={"RLB_TEST_MARK": mark})
    try:
        who = g.get_all_worker_results(g.run_all_workers_single_data("whoami"))
        assert [w["rank"] for w in who] == [0, 1, 2, 3] and all(w["world"] == 4 and w["tag"] == "hello" and w["group"] == "echo" for w in who)
        assert g.dp_size == 2 and g.get_dp_leader_worker_idx(1) == 2
        # only index 0 of an axis
        r = g.get_all_worker_results(g.run_all_workers_single_data("add", 1, y=1, run_rank_0_only_axes=["tensor_parallel"]))
        assert r == [2, 2002]
        # one entry per worker
        r = g.get_all_worker_results(g.run_all_workers_multiple_data("add", [1, 2, 3, 4], y=[10, 20, 30, 40]))
        assert r == [11, 1022, 2033, 3044]
        with pytest.raises(ValueError):
            g.run_all_workers_multiple_data("add", [1, 2])
        # sharded over data parallel, replicated over tensor parallel, one result per data-parallel index
        fut = g.run_all_workers_sharded_data("add", in_sharded_axes=["data_parallel"], replicate_on_axes=["tensor_parallel"],
                                             output_is_replicated=["tensor_parallel"], x=[5, 6], common_kwargs=dict(y=1))
        assert isinstance(fut, MultiWorkerFuture) and fut.called_workers == [0, 1, 2, 3] and fut.return_from_workers == [0, 2]
        assert g.get_all_worker_results(fut) == [6, 2007]
        # tensor parallel left free: only its index 0 is called; with dummy calls the others get None arguments
        fut = g.run_all_workers_sharded_data("add", in_sharded_axes=["data_parallel"], x=[7, 8])
        assert fut.called_workers == [0, 2] and g.get_all_worker_results(fut) == [7, 2008]
        fut = g.run_all_workers_sharded_data("add", in_sharded_axes=["data_parallel"], x=[7, 8], make_dummy_calls_to_free_axes=True)
        assert fut.called_workers == [0, 1, 2, 3] and g.get_all_worker_results(fut) == [7, 2008]
        with pytest.raises(ValueError):
            g.run_all_workers_sharded_data("add", in_sharded_axes=["data_parallel"], replicate_on_axes=["data_parallel"], x=[1, 2])
        # calls reach a worker in issue order
        hist = g.run_single_worker_single_data("history", 1).result()
        assert [h[1] for h in hist] == [2, 5, None]
        # a failure carries the worker's traceback; the group stays usable
        with pytest.raises(WorkerError) as e:
            g.get_all_worker_results(g.run_all_workers_single_data("boom"))
        assert "bad input on rank" in e.value.remote_traceback and e.value.method == "boom"
        # the workers form their own process group from the environment the group gave them
        assert g.get_all_worker_results(g.run_all_workers_single_data("all_reduce_rank")) == [10.0] * 4
    finally:
        assert g.shutdown(cleanup_method="cleanup", timeout=30)
    assert all(os.path.exists(f"{mark}.{r}") for r in range(4))
    assert all(w.proc.exitcode == 0 for w in g.workers)
    # the bundles are free again
    g2 = WorkerGroup(cluster, WorkerBuilder(EchoWorker, "again"), name="echo2")
    assert g2.get_all_worker_results(g2.run_all_workers_single_data("whoami"))[0]["tag"] == "again"
    g2.shutdown()


def test_worker_group_reports_a_constructor_failure():
    cluster = VirtualCluster([2], use_gpus=False)
    with pytest.raises(WorkerError) as e:
        WorkerGroup(cluster, WorkerBuilder(EchoWorker, "x", fail_on_rank=1), name="bad")
    assert "cannot build" in e.value.remote_traceback
    WorkerGroup(cluster, WorkerBuilder("test_worker_groups.EchoWorker", "by-name"), name="ok").shutdown()    # the claim was released


def _policy_cfg(**over):
    c = dict(model_name="tiny-llama-oracle", precision="float32", train_global_batch_size=4, train_micro_batch_size=2, max_total_sequence_length=64,
             max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-3)),
             generation=dict(max_new_tokens=5, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8))
    c.update(over)
    return c


def _policy_data():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 2048, (8, 20), generator=g)
    lens = torch.tensor([20, 13, 17, 20, 9, 20, 15, 11])
    return BatchedDataDict(input_ids=ids, input_lengths=lens, token_mask=(torch.arange(20)[None] < lens[:, None]).float(), sample_mask=torch.ones(8))


@pytest.mark.parametrize("par", [dict(), dict(tensor_parallel_size=2)])
def test_policy_facade_matches_an_in_process_worker(par, tmp_path):
    """The controller's policy over two worker processes (data parallel, or one tensor-parallel replica) gives what one
    in-process worker gives: log-probabilities, two optimizer steps, reference log-probabilities, a checkpoint."""
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.lm_policy import Policy
    from rl_b200.policy.worker import PolicyWorker

    data = _policy_data()
    reset_parallel()
    solo = PolicyWorker(_policy_cfg(), device="cpu", init_reference_model=True, seed=5)
    lp0 = solo.get_logprobs(data)["logprobs"]
    losses = [float(solo.train(data, NLLLossFn())["loss"][-1]) for _ in range(2)]
    lp2 = solo.get_logprobs(data)["logprobs"]
    cluster = VirtualCluster([2], use_gpus=False, name="policy")
    pol = Policy(cluster, _policy_cfg(parallel=par), init_reference_model=True, seed=5, backend="gloo")
    try:
        lay = pol.layouts()
        assert [l["rank"] for l in lay] == [0, 1] and lay[1]["tp_rank"] == (1 if par else 0) and pol.dp == (1 if par else 2)
        assert torch.allclose(pol.get_logprobs(data)["logprobs"], lp0, atol=2e-5)
        got = []
        for _ in range(2):
            r = pol.train(data, NLLLossFn())
            got.append(float(r["loss"][-1]))
            assert len(r["all_mb_metrics"]["loss"]) == 4          # 2 global batches x 2 micro-batches in total, whatever the layout
        assert got == pytest.approx(losses, rel=1e-4)
        assert torch.allclose(pol.get_logprobs(data)["logprobs"], lp2, atol=5e-5)
        assert torch.allclose(pol.get_reference_policy_logprobs(data)["reference_logprobs"], lp0, atol=2e-5)
        assert pol.prepare_for_generation()
        out = pol.generate(data, greedy=True)
        pol.finish_generation()
        assert out["output_ids"].shape[0] == 8 and (out["generation_lengths"] == 5).all()
        pol.save_checkpoint(str(tmp_path / "w"))
        assert os.path.exists(tmp_path / "w" / "config.json")
    finally:
        assert pol.shutdown()


def test_teacher_worker_group_scores_like_the_in_process_teacher():
    """A non-colocated teacher (its own worker group, tensor parallel 2) answers with the log-probabilities the in-process teacher
    gives; aliases that share a checkpoint share the group."""
    from dataclasses import asdict

    from rl_b200.algorithms import opd
    from rl_b200.models.config import preset
    from rl_b200.parallel.state import reset_parallel

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    master = dict(policy=_policy_cfg(), cluster=dict(backend="gloo"),
                  grpo=dict(adv_estimator=dict(name="opd")),
                  on_policy_distillation=dict(teacher_model_by_agent_name={"math": "tiny-llama-oracle", "code": "tiny-llama-oracle"},
                                              non_colocated_teachers=dict(enabled=True, default_teacher_cfg=dict(
                                                  num_nodes=1, gpus_per_node=2, tensor_model_parallel_size=2, precision="float32"))))
    data = _policy_data()
    reset_parallel()
    solo = opd.TeacherGroup(opd.create_teacher_configs(opd.opd_cfg(master))[0], master["policy"], model_cfg=mc)
    want = solo.get_logprobs(data)["reference_logprobs"]
    groups, alias_map = opd.create_teacher_groups(master, model_cfg=mc)
    try:
        assert list(groups) == ["math"] and alias_map == {"math": "math", "code": "math"}
        g = groups["math"]
        assert g.cluster.world_size() == 2 and g.policy.dp == 1 and [l["tp"] for l in g.policy.layouts()] == [2, 2]
        got = g.get_logprobs(data)["reference_logprobs"]
        assert torch.allclose(got, want, atol=3e-5)
        top = g.get_topk_logits(data, 4)
        assert top["topk_logits"].shape[0] == 8 and top["topk_indices"].shape[-1] == 4
    finally:
        for g in groups.values():
            assert g.shutdown()


class _RefitPeer:
    """Rank 0 hosts a trainer, rank 1 a generation service with different weights; neither joins a default process group."""

    def __init__(self, port):
        from rl_b200.models.config import preset
        from rl_b200.parallel.state import reset_parallel
        from rl_b200.policy.worker import PolicyWorker

        self.rank, self.port = int(os.environ["RANK"]), port
        reset_parallel()
        mc = preset("tiny-llama-oracle", torch_dtype="float32")
        self.worker = PolicyWorker(_policy_cfg(), model_cfg=mc, device="cpu", init_reference_model=False, init_optimizer=False, seed=11 + self.rank)
        self.gen = self.worker.build_generation() if self.rank == 1 else None

    def logprobs(self, data):
        return self.worker.get_logprobs(data)["logprobs"]

    def connect(self):
        if self.rank == 0:
            self.worker.init_collective("127.0.0.1", self.port, 2, train_world_size=1)
            return self.worker.prepare_refit_info()
        self.gen.init_collective(0, "127.0.0.1", self.port, 2, train_world_size=1)
        return None

    def refit(self, info=None):
        if self.rank == 0:
            return self.worker.broadcast_weights_for_collective(bucket_bytes=1 << 18)      # several buckets
        self.gen.prepare_refit_info(info)
        return self.gen.update_weights_from_collective()

    def generate(self, data):
        self.gen.prepare_for_generation()
        out = self.gen.generate(data, greedy=True)
        self.gen.finish_generation()
        return out["output_ids"]


def test_weights_reach_an_engine_outside_the_trainers_job():
    """The reference's collective refit interface: a trainer process and a generation process that share no process group meet
    on a communicator of their own, the trainer broadcasts packed buckets, the engine's weights become the trainer's."""
    from rl_b200.distributed.virtual_cluster import free_port

    data = _policy_data()
    g = WorkerGroup(VirtualCluster([2], use_gpus=False), WorkerBuilder(_RefitPeer, free_port()), name="refit")
    try:
        before = g.get_all_worker_results(g.run_all_workers_single_data("logprobs", data))
        assert not torch.allclose(before[0], before[1], atol=1e-3)                     # different seeds, different policies
        info = g.get_all_worker_results(g.run_all_workers_single_data("connect"))[0]
        assert "model.embed_tokens.weight" in info or len(info) > 0
        sent, ok = g.get_all_worker_results(g.run_all_workers_multiple_data("refit", [None, info]))
        assert sent > 1_000_000 and ok is True
        after = g.get_all_worker_results(g.run_all_workers_single_data("logprobs", data))
        assert torch.allclose(after[0], after[1], atol=1e-6) and torch.allclose(after[0], before[0], atol=1e-6)
        out = g.run_single_worker_single_data("generate", 1, data).result()
        assert out.shape[0] == 8
    finally:
        g.shutdown()
