"""Sequence packers and BatchedDataDict sharding / micro-batching."""

import random

import pytest
import torch

from rl_b200.data.packing import get_packer
from rl_b200.distributed.batched_data_dict import BatchedDataDict

ALGOS = ["concatenative", "first_fit", "first_fit_decreasing", "first_fit_shuffle", "modified_first_fit_decreasing"]


@pytest.mark.parametrize("algo", ALGOS)
def test_packers_are_valid_partitions(algo):
    rng = random.Random(0)
    lens = [rng.randint(1, 1000) for _ in range(500)]
    p = get_packer(algo, 1024, collect_metrics=True)
    bins = p.pack(lens)
    flat = sorted(i for b in bins for i in b)
    assert flat == list(range(len(lens)))
    assert all(sum(lens[i] for i in b) <= 1024 for b in bins)
    assert p.metrics.aggregated()["total_sequences"] == 500


def test_mffd_no_worse_than_ffd_on_classic_case():
    lens = [51] * 6 + [27] * 6 + [26] * 6 + [23] * 12
    ffd = len(get_packer("first_fit_decreasing", 100).pack(lens))
    mffd = len(get_packer("modified_first_fit_decreasing", 100).pack(lens))
    lower = -(-sum(lens) // 100)
    assert lower <= mffd <= ffd


def test_packer_rejects_oversize_and_pads_bin_count():
    with pytest.raises(ValueError):
        get_packer("first_fit", 10).pack([11])
    bins = get_packer("first_fit_decreasing", 100, min_bin_count=4, bin_count_multiple=4).pack([60, 30, 20])
    assert len(bins) % 4 == 0 and sorted(i for b in bins for i in b) == [0, 1, 2]


def _data(n=16, S=12):
    lens = torch.randint(2, S + 1, (n,), generator=torch.Generator().manual_seed(0))
    return BatchedDataDict(input_ids=torch.arange(n * S).reshape(n, S), input_lengths=lens, tag=[f"s{i}" for i in range(n)])


def test_shard_plain_and_uneven():
    d = _data()
    shards = d.shard_by_batch_size(4, batch_size=8)
    assert [s.size for s in shards] == [4, 4, 4, 4]
    # every global batch of 8 is split evenly: shard r holds samples r*2..r*2+1 of batch 0 and of batch 1
    assert shards[1]["tag"] == ["s2", "s3", "s10", "s11"]
    un = d.slice(0, 10).shard_by_batch_size(4, allow_uneven_shards=True)
    assert [s.size for s in un] == [3, 3, 2, 2]


def test_dynamic_batching_respects_budget_and_roundtrips():
    d = _data(32, 64)
    shards, order = d.shard_by_batch_size(2, batch_size=16, dynamic_batching_args=dict(
        input_key="input_ids", input_lengths_key="input_lengths", sequence_length_round=8, max_tokens_per_microbatch=128))
    assert sorted(order) == list(range(32))
    for sh in shards:
        n = 0
        for mb in sh.make_microbatch_iterator_with_dynamic_shapes():
            assert mb["input_ids"].shape[0] * mb["input_ids"].shape[1] <= 128 or mb["input_ids"].shape[0] == 1
            assert int(mb["input_lengths"].max()) <= mb["input_ids"].shape[1]
            n += mb.size
        assert n == sh.size
    merged = BatchedDataDict.from_batches(shards).reorder_data(order)
    assert merged["tag"] == d["tag"] and torch.equal(merged["input_ids"], d["input_ids"])


def test_sequence_packing_bins():
    d = _data(32, 64)
    shards, order = d.shard_by_batch_size(4, batch_size=32, sequence_packing_args=dict(
        input_key="input_ids", input_lengths_key="input_lengths", max_tokens_per_microbatch=160, algorithm="modified_first_fit_decreasing"))
    counts = {sh.get_microbatch_iterator_len() for sh in shards}
    assert len(counts) == 1  # every rank steps the same number of micro-batches
    assert sorted(order) == list(range(32))
    for sh in shards:
        for mb in sh.make_microbatch_iterator_for_packable_sequences():
            assert int(mb["input_lengths"].sum()) <= 160


def test_from_batches_pads_and_repeat_interleave():
    a = BatchedDataDict(x=torch.ones(2, 3), l=[1, 2])
    b = BatchedDataDict(x=torch.ones(1, 5), l=[3])
    m = BatchedDataDict.from_batches([a, b], pad_value_dict={"x": -1})
    assert m["x"].shape == (3, 5) and m["x"][0, 4] == -1 and m["l"] == [1, 2, 3]
    r = m.repeat_interleave(2)
    assert r.size == 6 and r["l"] == [1, 1, 2, 2, 3, 3]


def test_local_dataset_rows_of_the_registry(tmp_path):
    """Sets that live in local files: jsonl with key renames, Arrow / Parquet text corpora, gym-style records."""
    import json

    import pyarrow as pa
    import pyarrow.parquet as pq

    from rl_b200.data.datasets.registry import HF_SETS, load_raw_dataset
    from rl_b200.data.processors import get_processor

    p = tmp_path / "intent.jsonl"
    p.write_text("\n".join(json.dumps(dict(text=f"q{i}", label=str(i))) for i in range(3)))
    recs, proc = load_raw_dataset(dict(dataset_name="intent", data_path=str(p)))
    assert len(recs) == 3 and recs[1]["problem"] == "q1" and recs[1]["expected_answer"] == "1" and proc == "math_data_processor"
    table = pa.table({"messages": [[{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]] * 4})
    pq.write_table(table, tmp_path / "c.parquet")
    with pa.OSFile(str(tmp_path / "c.arrow"), "wb") as f, pa.ipc.new_file(f, table.schema) as w:
        w.write_table(table)
    for name in ("c.parquet", "c.arrow"):
        recs, proc = load_raw_dataset(dict(dataset_name="arrow_text", data_path=str(tmp_path / name), max_samples=3))
        assert len(recs) == 3 and recs[0]["messages"][1]["content"] == "yo" and proc == "sft_processor"
    assert load_raw_dataset(dict(dataset_name="local_math", data_path=str(p), problem_key="text", solution_key="label"))[0][2]["expected_answer"] == "2"
    for name, row in HF_SETS.items():
        get_processor(row[5])     # every row names a registered processor
    assert {"OpenR1-Math-220k", "geometry3k", "refcoco", "avqa", "MMAU", "nemogym", "BinaryPreferenceDataset"} <= set(HF_SETS)


def test_message_log_decompose_and_reconstruct_round_trip():
    from rl_b200.data.llm_message_utils import (attach_message_log_view, batched_message_log_to_flat_message, decompose_message_log,
                                                get_first_index_that_differs, message_log_shape, pad_tensor, remap_dataset_keys,
                                                validate_tensor_consistency)
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    logs = [[{"role": "user", "content": "hi", "token_ids": torch.tensor([1, 2, 3])},
             {"role": "assistant", "content": "yo", "token_ids": torch.tensor([4, 5]), "generation_logprobs": torch.tensor([-0.1, -0.2])},
             {"role": "environment", "content": "ok", "token_ids": torch.tensor([6])},
             {"role": "assistant", "content": "bye", "token_ids": torch.tensor([7, 8, 9]), "generation_logprobs": torch.tensor([-0.3, -0.4, -0.5])}],
            [{"role": "system", "content": "no tokens"},
             {"role": "user", "content": "q", "token_ids": torch.tensor([10])},
             {"role": "assistant", "content": "a", "token_ids": torch.tensor([11, 12]), "generation_logprobs": torch.tensor([-1.0, -2.0])}]]
    assert message_log_shape(logs[0])[1] == {"token_ids": torch.Size([2]), "generation_logprobs": torch.Size([2])}
    d = decompose_message_log(logs)
    assert d["turn_lengths"].tolist() == [[3, 2, 1, 3], [0, 1, 2, 0]] and d["response_token_lengths"].tolist() == [2, 2]
    assert d["turn_roles"][1] == ["system", "user", "assistant"]
    for log in logs:
        for m in log:
            if "token_ids" in m and "generation_logprobs" not in m:
                m["generation_logprobs"] = torch.zeros(m["token_ids"].numel())
    flat, lens = batched_message_log_to_flat_message([[m for m in log if "token_ids" in m] for log in logs], {"token_ids": 0})
    batch = BatchedDataDict(input_ids=flat["token_ids"], generation_logprobs=flat["generation_logprobs"], **{k: d[k] for k in
                                                                                                           ("turn_lengths", "turn_roles", "turn_contents")})
    attach_message_log_view(batch)
    back = batch["message_log"]
    assert [m["role"] for m in back[1]] == ["system", "user", "assistant"] and "token_ids" not in back[1][0]
    assert back[0][3]["token_ids"].tolist() == [7, 8, 9] and back[0][3]["generation_logprobs"].tolist() == pytest.approx([-0.3, -0.4, -0.5])
    assert "generation_logprobs" not in back[0][2]
    assert back[0][1]["token_ids"].data_ptr() == batch["input_ids"][0, 3:].data_ptr()       # a view, not a copy
    assert get_first_index_that_differs("abcX", "abcY") == 3 and get_first_index_that_differs("ab", "abc") == 2
    assert pad_tensor(torch.tensor([1, 2]), 4, "left", 9).tolist() == [9, 9, 1, 2] and pad_tensor(torch.tensor([1, 2]), 1).tolist() == [1, 2]
    with pytest.raises(ValueError):
        validate_tensor_consistency([torch.zeros(2, dtype=torch.long), torch.zeros(2)])
    assert remap_dataset_keys([{"q": 1, "a": 2, "z": 3}], {"q": "input", "a": "output"}) == [{"z": 3, "input": 1, "output": 2}]


def test_formatted_message_log_applies_task_prompts_and_generation_headers():
    from rl_b200.data.interfaces import TaskDataSpec
    from rl_b200.data.llm_message_utils import get_formatted_message_log
    from rl_b200.data.tokenizers import ByteTokenizer

    tok = ByteTokenizer()
    spec = TaskDataSpec(task_name="t", prompt="Solve: {}", system_prompt="Be brief.")
    log = get_formatted_message_log([{"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"}, {"role": "user", "content": "3+3?"}],
                                    tok, spec, add_eos_token=False, add_generation_prompt=True)
    text = "".join(tok.decode(m["token_ids"]) for m in log)
    assert [m["role"] for m in log] == ["system", "user", "assistant", "user"]
    assert text == "<bos><|system|>Be brief.<|end|><|user|>Solve: 2+2?<|end|><|assistant|>4<|end|><|user|>3+3?<|end|><|assistant|>"
    # the assistant header rendered after the first user message belongs to that message; the assistant turn owns only its text
    assert tok.decode(log[1]["token_ids"]).endswith("<|assistant|>") and tok.decode(log[2]["token_ids"]) == "4<|end|>"
    # multimodal content: text parts are replaced by the rendered chunk, other parts stay
    mm = get_formatted_message_log([{"role": "user", "content": [{"type": "text", "text": "what is this?"}, {"type": "image", "image": "x.png"}]}],
                                   _ListContentTokenizer(), None)
    assert mm[0]["content"][1] == {"type": "image", "image": "x.png"} and "what is this?" in mm[0]["content"][0]["text"]


class _ListContentTokenizer:
    """A byte tokenizer whose template accepts typed content lists (what multimodal processors do)."""

    def __init__(self):
        from rl_b200.data.tokenizers import ByteTokenizer

        self.t = ByteTokenizer()
        self.bos_token, self.eos_token = self.t.bos_token, self.t.eos_token

    def apply_chat_template(self, msgs, **kw):
        flat = [dict(m, content="".join(p.get("text", "<image>") for p in m["content"]) if isinstance(m["content"], list) else m["content"]) for m in msgs]
        return self.t.apply_chat_template(flat, **kw)

    def __call__(self, *a, **k):
        return self.t(*a, **k)
