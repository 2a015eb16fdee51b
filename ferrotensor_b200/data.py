"""The data side of the step: examples, datasets, batches (ferrotensor-trainer/src/data.rs).

`TrainingExample` (data.rs:33-98: next-token and response-masked SFT examples), `TextDataset`
(:100-260: sequences, packed token streams, `.bin` files of little-endian u32 ids, greedy
packing), `sft_example_from_tokens` (the length rules of `build_sft_example`, :263-300, on
already tokenised text: no tokenizer ships with this library), `DataLoader` (:344-512: batches
right-padded with the pad token, attention and loss masks, Fisher-Yates shuffle driven by the
reference's 64-bit LCG so that a seed and an epoch give the reference's order) and
`supervised_tokens` / the token-weighted evaluation mean (cli main.rs:1099-1137).
The `Batch` produced here is the one `Trainer.train_batch` consumes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

from .trainer import Batch

_MASK64 = (1 << 64) - 1


@dataclass
class TrainingExample:
    input_ids: List[int]
    target_ids: List[int]
    loss_mask: List[int]

    @staticmethod
    def from_next_token(sequence: Sequence[int]) -> "TrainingExample":
        """Inputs are all but the last token, targets all but the first, all supervised."""
        seq = [int(t) for t in sequence]
        if len(seq) < 2:
            return TrainingExample(list(seq), list(seq), [1] * len(seq))
        return TrainingExample(seq[:-1], seq[1:], [1] * (len(seq) - 1))

    @staticmethod
    def from_sft_prompt_response(prompt_tokens: Sequence[int], response_tokens: Sequence[int]) -> "TrainingExample":
        """Loss only where the prediction recovers a response token: the first response token is
        `full[len(prompt)]`, so its target index is `len(prompt) - 1`."""
        prompt, response = [int(t) for t in prompt_tokens], [int(t) for t in response_tokens]
        full = prompt + response
        if len(full) < 2:
            return TrainingExample.from_next_token(full)
        target = full[1:]
        if prompt and response:
            first = max(len(prompt) - 1, 0)
            mask = [0] * first + [1] * (len(target) - first)
        else:
            mask = [1] * len(target)
        return TrainingExample(full[:-1], target, mask)


def sft_example_from_tokens(prompt_tokens: Sequence[int], response_tokens: Sequence[int],
                            max_len: int) -> Optional[TrainingExample]:
    """`build_sft_example` after tokenisation: truncated at the end to `max_len` inputs (the prompt
    is kept whole); dropped (None) when either side is empty, the prompt alone exceeds `max_len`,
    or no supervised target survives."""
    if not len(prompt_tokens) or not len(response_tokens):
        return None
    if max_len < 2 or len(prompt_tokens) > max_len:
        return None
    ex = TrainingExample.from_sft_prompt_response(prompt_tokens, response_tokens)
    if len(ex.input_ids) > max_len:
        ex = TrainingExample(ex.input_ids[:max_len], ex.target_ids[:max_len], ex.loss_mask[:max_len])
    if len(ex.input_ids) < 2 or 1 not in ex.loss_mask:
        return None
    return ex


def pack_windows(sequences: Iterable[Sequence[int]], max_len: int) -> List[List[int]]:
    """Greedy packing into windows of at most `max_len` tokens (data.rs:529-560): longer
    sequences are cut into `max_len` pieces, a window closes when the next piece would not fit,
    a single leftover token that cannot be joined is dropped."""
    packed: List[List[int]] = []
    if max_len < 2:
        return packed
    current: List[int] = []
    for seq in sequences:
        seq = list(seq)
        for s in range(0, len(seq), max_len):
            piece = seq[s:s + max_len]
            if len(current) + len(piece) > max_len:
                if len(current) >= 2:
                    packed.append(current)
                current = []
            current = current + piece
    if len(current) >= 2:
        packed.append(current)
    return packed


class TextDataset:
    def __init__(self):
        self.samples: List[TrainingExample] = []

    def add_sample(self, input_ids: Sequence[int], target_ids: Sequence[int]) -> None:
        self.samples.append(TrainingExample(list(input_ids), list(target_ids), [1] * len(target_ids)))

    def add_example(self, example: TrainingExample) -> None:
        self.samples.append(example)

    @staticmethod
    def from_sequences(sequences: Iterable[Sequence[int]]) -> "TextDataset":
        ds = TextDataset()
        ds.samples = [TrainingExample.from_next_token(s) for s in sequences]
        return ds

    @staticmethod
    def from_packed_tokens(tokens: Sequence[int], sequence_length: int) -> "TextDataset":
        """Windows of `sequence_length` tokens, stride `sequence_length - 1` (data.rs:221-237)."""
        ds = TextDataset()
        if sequence_length < 2 or len(tokens) < sequence_length:
            return ds
        stride = max(sequence_length - 1, 1)
        start = 0
        while start + sequence_length <= len(tokens):
            ds.samples.append(TrainingExample.from_next_token(tokens[start:start + sequence_length]))
            start += stride
        return ds

    @staticmethod
    def from_token_bin(path, sequence_length: int) -> "TextDataset":
        raw = Path(path).read_bytes()
        tokens = np.frombuffer(raw[:len(raw) // 4 * 4], dtype="<u4")
        return TextDataset.from_packed_tokens(tokens.tolist(), sequence_length)

    @staticmethod
    def pack_sequences(sequences: Iterable[Sequence[int]], max_len: int) -> "TextDataset":
        return TextDataset.from_sequences(pack_windows(sequences, max_len))

    def examples(self) -> List[TrainingExample]:
        return self.samples

    def __len__(self) -> int:
        return len(self.samples)

    def is_empty(self) -> bool:
        return not self.samples

    def get(self, idx: int) -> Tuple[List[int], List[int]]:
        return self.samples[idx].input_ids, self.samples[idx].target_ids

    def get_loss_mask(self, idx: int) -> Optional[List[int]]:
        return self.samples[idx].loss_mask


def supervised_tokens(ds: TextDataset) -> int:
    return sum(sum(1 for m in e.loss_mask if m != 0) for e in ds.examples())


class SimpleRng:
    """data.rs:514-527: the 64-bit LCG behind the shuffle."""

    def __init__(self, seed: int):
        self.state = (int(seed) + 1) & _MASK64

    def next(self) -> int:
        self.state = (self.state * 6364136223846793005 + 1) & _MASK64
        return self.state


class DataLoader:
    """Batches of `batch_size` examples in index order (or the seeded shuffle of it)."""

    def __init__(self, dataset: TextDataset, batch_size: int, shuffle: bool, pad_token_id: int = 0,
                 indices: Optional[Sequence[int]] = None):
        self.dataset, self.batch_size = dataset, max(int(batch_size), 1)
        self.pad_token_id, self.shuffle = int(pad_token_id), bool(shuffle)
        self.base_indices = list(range(len(dataset))) if indices is None else [int(i) for i in indices]
        self.indices = list(self.base_indices)
        self.current_idx = 0
        self.seed: Optional[int] = None
        self.epoch = 0

    def with_seed(self, seed: int) -> "DataLoader":
        self.seed = int(seed) & _MASK64
        return self

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    def reset(self) -> None:
        """Rewind; with shuffling, the order of (seed, epoch): seed ^ epoch * 0x9E3779B97F4A7C15."""
        self.current_idx = 0
        self.indices = list(self.base_indices)
        if self.shuffle:
            if self.seed is not None:
                seed = self.seed ^ ((self.epoch * 0x9E3779B97F4A7C15) & _MASK64)
            else:
                import time
                seed = time.time_ns() & _MASK64
            rng = SimpleRng(seed)
            for i in range(len(self.indices) - 1, 0, -1):
                j = (rng.next() >> 33) % (i + 1)
                self.indices[i], self.indices[j] = self.indices[j], self.indices[i]

    def num_batches(self) -> int:
        return -(-len(self.indices) // self.batch_size)

    def __len__(self) -> int:
        return len(self.indices)

    def is_empty(self) -> bool:
        return not self.indices

    def __iter__(self) -> Iterator[Batch]:
        return self

    def __next__(self) -> Batch:
        if self.current_idx >= len(self.indices):
            raise StopIteration
        end = min(self.current_idx + self.batch_size, len(self.indices))
        picked = self.indices[self.current_idx:end]
        inputs, targets, raw_masks = [], [], []
        longest = 0
        for idx in picked:
            inp, tgt = self.dataset.get(idx)
            mask = self.dataset.get_loss_mask(idx)
            if mask is None:
                mask = [1] * len(tgt)
            longest = max(longest, len(inp), len(tgt))
            inputs.append(list(inp)); targets.append(list(tgt)); raw_masks.append(list(mask))
        p_in, p_tg, attn, loss = [], [], [], []
        for inp, tgt, mask in zip(inputs, targets, raw_masks):
            valid = min(len(inp), len(tgt))
            p_in.append((inp + [self.pad_token_id] * longest)[:longest])
            p_tg.append((tgt + [self.pad_token_id] * longest)[:longest])
            attn.append([1] * valid + [0] * (longest - valid))
            row = [0] * longest
            for i in range(min(valid, len(mask))):
                row[i] = int(mask[i])
            loss.append(row)
        self.current_idx = end
        return Batch(padded_input_ids=p_in, padded_target_ids=p_tg, attention_mask=attn, loss_masks=loss,
                     input_ids=inputs, target_ids=targets, max_seq_len=longest)
