"""Data side of the step: the reference's unit tests (ferrotensor-trainer/src/data.rs:562-702)
restated, the shuffle order pinned against an independent big-integer restatement of its LCG,
and the evaluation mean against the oracle on the GPU."""

import copy

import numpy as np
import pytest

from ferrotensor_b200.data import (DataLoader, SimpleRng, TextDataset, TrainingExample, pack_windows,
                                   sft_example_from_tokens, supervised_tokens)


def test_text_dataset():
    ds = TextDataset.from_sequences([[1, 2, 3, 4], [5, 6, 7, 8]])
    assert len(ds) == 2
    assert ds.get(0) == ([1, 2, 3], [2, 3, 4])
    assert ds.get_loss_mask(0) == [1, 1, 1]
    one = TrainingExample.from_next_token([7])
    assert (one.input_ids, one.target_ids, one.loss_mask) == ([7], [7], [1])


def test_sft_example_masks_only_response_tokens():
    ex = TrainingExample.from_sft_prompt_response([10, 11, 12], [20, 21])
    assert ex.input_ids == [10, 11, 12, 20]
    assert ex.target_ids == [11, 12, 20, 21]
    assert ex.loss_mask == [0, 0, 1, 1]
    assert TrainingExample.from_sft_prompt_response([], [1, 2, 3]).loss_mask == [1, 1]


def test_sft_length_rules():
    assert sft_example_from_tokens([], [1], 8) is None and sft_example_from_tokens([1], [], 8) is None
    assert sft_example_from_tokens([1, 2, 3], [4], 2) is None          # prompt alone exceeds max_len
    assert sft_example_from_tokens([1, 2, 3], [4], 1) is None
    ex = sft_example_from_tokens([1, 2, 3], [4, 5, 6, 7], 4)            # truncated at the end
    assert ex.input_ids == [1, 2, 3, 4] and ex.target_ids == [2, 3, 4, 5] and ex.loss_mask == [0, 0, 1, 1]
    ex = sft_example_from_tokens([1, 2, 3], [4, 5], 3)                  # one supervised target survives
    assert ex.input_ids == [1, 2, 3] and ex.loss_mask == [0, 0, 1]
    assert sft_example_from_tokens([1], [2], 8) is None               # a single input token is dropped
    assert sft_example_from_tokens([1], [2, 3], 8).loss_mask == [1, 1]


def test_dataloader_batching():
    ds = TextDataset.from_sequences([[1, 2], [3, 4], [5, 6], [7, 8], [9, 10]])
    assert DataLoader(ds, 2, False).num_batches() == 3
    assert [b.batch_size for b in DataLoader(ds, 2, False)] == [2, 2, 1]


def test_dataloader_pads_and_masks_batches():
    ds = TextDataset.from_sequences([[1, 2, 3, 4], [5, 6, 7]])
    batch = next(DataLoader(ds, 2, False, pad_token_id=99))
    assert batch.max_seq_len == 3
    assert batch.padded_input_ids[0] == [1, 2, 3]
    assert batch.padded_input_ids[1] == [5, 6, 99]
    assert batch.padded_target_ids[1] == [6, 7, 99]
    assert batch.attention_mask[0] == [1, 1, 1] and batch.attention_mask[1] == [1, 1, 0]
    assert batch.loss_masks[1] == [1, 1, 0]
    assert batch.input_ids[1] == [5, 6]


def test_packed_bin_and_txt_share_next_token_mask_semantics(tmp_path):
    packed = TextDataset.from_packed_tokens([1, 2, 3, 4, 5, 6], 4)
    assert not packed.is_empty()
    for i in range(len(packed)):
        inp, tgt = packed.get(i)
        mask = packed.get_loss_mask(i)
        assert all(m == 1 for m in mask) and len(inp) == len(tgt) == len(mask)
    assert TextDataset.from_sequences([[9, 8, 7, 6]]).get_loss_mask(0) == [1, 1, 1]
    # windows of 4 with stride 3: [1..4], [4..7]; a .bin file of little-endian u32 gives the same
    seven = TextDataset.from_packed_tokens(list(range(1, 8)), 4)
    assert [e.input_ids for e in seven.examples()] == [[1, 2, 3], [4, 5, 6]]
    path = tmp_path / "tokens.bin"
    path.write_bytes(np.arange(1, 8, dtype="<u4").tobytes() + b"\x01")     # a trailing odd byte is ignored
    from_bin = TextDataset.from_token_bin(path, 4)
    assert [e.target_ids for e in from_bin.examples()] == [e.target_ids for e in seven.examples()]
    assert TextDataset.from_packed_tokens([1, 2, 3], 4).is_empty() and TextDataset.from_packed_tokens([1, 2], 1).is_empty()


def test_sft_dataloader_preserves_response_mask_under_padding():
    ds = TextDataset()
    ds.add_example(TrainingExample.from_sft_prompt_response([1, 2, 3], [4, 5]))
    ds.add_example(TrainingExample.from_sft_prompt_response([10, 11], [12]))
    batch = next(DataLoader(ds, 2, False, pad_token_id=0))
    assert sum(batch.loss_masks[0]) == 2 and batch.loss_masks[0][:2] == [0, 0]
    assert 1 in batch.loss_masks[1] and 0 in batch.loss_masks[1]
    assert supervised_tokens(ds) == 3


def test_pack_windows():
    tokens = list(range(5000))
    windows = pack_windows([tokens], 256)
    assert len(windows) == 20 and all(len(w) <= 256 for w in windows)
    assert [t for w in windows for t in w] == tokens
    assert pack_windows([[1, 2], [3, 4], [5, 6, 7]], 4) == [[1, 2, 3, 4], [5, 6, 7]]
    assert pack_windows([[1, 2], [3, 4, 5, 6, 7, 8, 9]], 3) == [[1, 2], [3, 4, 5], [6, 7, 8]]
    assert pack_windows([[1], [2, 3, 4]], 3) == [[2, 3, 4]]
    assert pack_windows([[], [1, 2]], 4) == [[1, 2]]
    assert pack_windows([[1, 2, 3], [4, 5]], 1) == []
    ds = TextDataset.pack_sequences([list(range(10))], 4)
    assert len(ds.examples()) == len(pack_windows([list(range(10))], 4)) == 3


def _reference_order(n, seed, epoch):
    """data.rs:409-430 with Python integers: state = seed' + 1; x -> x * 6364136223846793005 + 1
    (mod 2^64); Fisher-Yates from the back with j = (x >> 33) % (i + 1)."""
    m = (1 << 64) - 1
    state = ((seed ^ ((epoch * 0x9E3779B97F4A7C15) & m)) + 1) & m
    idx = list(range(n))
    for i in range(n - 1, 0, -1):
        state = (state * 6364136223846793005 + 1) & m
        j = (state >> 33) % (i + 1)
        idx[i], idx[j] = idx[j], idx[i]
    return idx


def test_shuffle_order_is_the_reference_lcg():
    r = SimpleRng(0)
    assert r.next() == 6364136223846793006 and r.next() == (6364136223846793006 * 6364136223846793005 + 1) % (1 << 64)
    ds = TextDataset.from_sequences([[i, i + 1] for i in range(37)])
    loader = DataLoader(ds, 5, True).with_seed(42)
    orders = []
    for epoch in (0, 1, 0):
        loader.set_epoch(epoch)
        loader.reset()
        got = [b.padded_input_ids[k][0] for b in loader for k in range(b.batch_size)]
        assert got == _reference_order(37, 42, epoch)
        orders.append(got)
    assert orders[0] == orders[2] and orders[0] != orders[1] and sorted(orders[1]) == list(range(37))
    # one rank's shard (distributed.rs:222-227) keeps its own indices
    shard = DataLoader(ds, 4, False, indices=[i for i in range(37) if i % 4 == 1])
    assert [b.padded_input_ids[0][0] for b in shard][:3] == [1, 17, 33]


@pytest.mark.gpu
def test_evaluate_is_the_token_weighted_mean(cuda_ctx):
    """`evaluate` (cli main.rs:1111-1137) against the oracle's per-sequence losses; training on a
    loader's batches afterwards still starts from clean gradients."""
    import torch
    from oracle import lora_step as ol
    from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    from tests.test_step_gpu import _oracle_cfg, _oracle_params
    w = copy.deepcopy(WORKLOADS["tiny"])
    weights = init_weights(w.model, 4, f16_base=w.f16_base)
    adapters = init_adapters(w.model, w.lora, 4, b_std=0.02)
    rng = np.random.default_rng(1)
    ds = TextDataset()
    for n_prompt, n_resp in ((3, 5), (6, 2), (2, 9), (4, 4), (1, 1)):
        ds.add_example(TrainingExample.from_sft_prompt_response(rng.integers(0, w.model.vocab, n_prompt).tolist(),
                                                                rng.integers(0, w.model.vocab, n_resp).tolist()))
    model = LoraModel(cuda_ctx, w.model, w.lora, weights, adapters, f16_base=w.f16_base)
    tr = Trainer(model, AdamW(1e-3)).with_grad_accum_steps(2)
    tr.length_bucket = 4
    model.grads.fill_(3.0)
    loss, tokens = tr.evaluate(ds, limit=4, chunk=3)
    assert tokens == 5 + 2 + 9 + 4 and torch.all(model.grads == 3.0)
    ocfg = _oracle_cfg(w.model, w.lora, f16_base=w.f16_base)
    p = _oracle_params(w.model, weights, adapters, w.f16_base)
    total, count = 0.0, 0
    for e in ds.examples()[:4]:
        ids = np.asarray([e.input_ids], dtype=np.int64)
        r = ol.forward_backward(ocfg, p, ids, np.asarray([e.target_ids], dtype=np.int64),
                                np.asarray([e.loss_mask], dtype=np.uint8), seed_scale=1.0)
        (l, n), = r.per_sequence
        total += l * n
        count += n
    assert count == tokens and abs(loss - total / count) <= 1e-4 + 1e-3 * abs(total / count)
    assert tr.evaluate(TextDataset())[1] == 0 and np.isnan(tr.evaluate(TextDataset())[0])
    stats = []
    for batch in DataLoader(ds, 2, False):
        stats += tr.train_batch(batch)
    assert sum(1 for s in stats if s.optimizer_step) == 2
    model.close()
