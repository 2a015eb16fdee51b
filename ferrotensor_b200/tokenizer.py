"""Text to token ids for the data side of the step (ferrotensor-loader/src/tokenizer.rs).

The reference binds the Hugging Face `tokenizers` library; so does this wrapper (its Python
package), with the reference's rules around it: the special-token ids (tokenizer.rs:66-90: the
`bos_token` that `tokenizer_config.json` declares, else `<|im_start|>`, else `<s>`, else 1;
`<|im_end|>`, else `</s>`, else 2; `<pad>`, else 0), the plain `model.vocab` reader for a file
without a model `type` (:177-205), and the ChatML prompt of `conversation_prompt` (:238-250).
Nothing here touches the device.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Sequence


class TokenizerError(RuntimeError):
    pass


def _declared_bos_token(tokenizer_path: Path) -> Optional[str]:
    cfg_path = tokenizer_path.with_name("tokenizer_config.json")
    if not cfg_path.exists():
        return None
    try:
        cfg = json.loads(cfg_path.read_text())
    except (OSError, ValueError) as e:
        raise TokenizerError(f"Failed to parse {cfg_path}: {e}") from e
    bos = cfg.get("bos_token") if isinstance(cfg, dict) else None
    if isinstance(bos, str):
        return bos
    if isinstance(bos, dict) and isinstance(bos.get("content"), str):
        return bos["content"]
    return None


def conversation_prompt(system: Optional[str], turns: Sequence[str]) -> str:
    """An optional system turn, then `turns` alternating user and assistant (user first), then
    the assistant header, so that the model continues as the assistant."""
    parts = []
    if system is not None:
        parts.append(("system", system))
    parts += [(("user", "assistant")[i % 2], t) for i, t in enumerate(turns)]
    return "".join(f"<|im_start|>{role}\n{text}<|im_end|>\n" for role, text in parts) + "<|im_start|>assistant\n"


def chat_prompt(system: Optional[str], user: str) -> str:
    return conversation_prompt(system, [user])


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], bos: int, eos: int, pad: int, hf=None):
        self.vocab = vocab
        self.id_to_token = {i: t for t, i in vocab.items()}
        self.bos_token_id, self.eos_token_id, self.pad_token_id = bos, eos, pad
        self.hf_tokenizer = hf

    @staticmethod
    def from_file(path) -> "Tokenizer":
        path = Path(path)
        if not path.is_file():
            raise TokenizerError(f"Failed to read tokenizer.json: {path} is not a regular file")
        declared = _declared_bos_token(path)
        hf_error: Optional[Exception] = None
        try:
            import tokenizers
            hf = tokenizers.Tokenizer.from_file(str(path))
        except Exception as e:                      # the library's own error type, or its absence
            hf, hf_error = None, e
        if hf is not None:
            vocab = hf.get_vocab(True)
            if not vocab:
                raise TokenizerError(f"{path}: tokenizer vocabulary is empty")
            lookup = hf.token_to_id
        else:
            try:
                parsed = json.loads(path.read_text())
                model = parsed["model"]
                vocab = dict(model["vocab"])
            except (OSError, ValueError, KeyError, TypeError) as e:
                raise TokenizerError(f"Failed to parse {path}: {e}") from e
            if model.get("type") is not None:
                raise TokenizerError(f"{path}: cannot load the {model['type']} tokenizer: {hf_error}")
            if not vocab:
                raise TokenizerError(f"{path}: tokenizer vocabulary is empty")
            seen: Dict[int, str] = {}
            for tok, i in vocab.items():
                if i in seen:
                    raise TokenizerError(f"{path}: token id {i} is used by more than one token")
                seen[i] = tok
            lookup = vocab.get

        def first(names, default):
            for n in names:
                if n is None:
                    continue
                i = lookup(n)
                if i is not None:
                    return int(i)
            return default

        bos = first([declared, "<|im_start|>", "<s>"], 1)
        eos = first(["<|im_end|>", "</s>"], 2)
        pad = first(["<pad>"], 0)
        return Tokenizer({t: int(i) for t, i in vocab.items()}, bos, eos, pad, hf)

    def _encode_with(self, text: str, add_special_tokens: bool) -> List[int]:
        if self.hf_tokenizer is not None:
            try:
                return list(self.hf_tokenizer.encode(text, add_special_tokens=add_special_tokens).ids)
            except Exception as e:
                raise TokenizerError(f"tokenizer cannot encode the text: {e}") from e
        # no merges in a plain vocabulary map: whole words, then the word after a space, then
        # single characters, then <unk>
        out = [self.bos_token_id] if add_special_tokens else []
        unk = self.vocab.get("<unk>", 0)
        for word in text.split():
            if word in self.vocab:
                out.append(self.vocab[word])
            elif "Ġ" + word in self.vocab:
                out.append(self.vocab["Ġ" + word])
            else:
                out.extend(self.vocab.get(c, unk) for c in word)
        return out

    def encode(self, text: str) -> List[int]:
        """With the tokenizer's special tokens (a leading BOS when it defines one)."""
        return self._encode_with(text, True)

    def encode_continuation(self, text: str) -> List[int]:
        """Without special tokens: text that continues a sequence (an SFT response)."""
        return self._encode_with(text, False)

    def encode_chat(self, system: Optional[str], user: str) -> List[int]:
        return self.encode(chat_prompt(system, user))

    def decode(self, tokens: Sequence[int]) -> str:
        if self.hf_tokenizer is not None:
            try:
                return self.hf_tokenizer.decode([int(t) for t in tokens], skip_special_tokens=True)
            except Exception as e:
                raise TokenizerError(f"tokenizer cannot decode {len(tokens)} ids: {e}") from e
        out = ""
        for t in tokens:
            if t in (self.bos_token_id, self.eos_token_id, self.pad_token_id):
                continue
            tok = self.id_to_token.get(int(t))
            if tok is None:
                continue
            if tok.startswith("Ġ"):
                out += (" " if out else "") + tok[1:]
            else:
                out += tok
        return out


def byte_level_tokenizer_json() -> dict:
    """A `tokenizer.json` that encodes text as its UTF-8 bytes (tokenizer.rs:279-296): a BPE
    model without merges over <pad> 0, <s> 1, </s> 2 and the 256 stand-in characters of the
    ByteLevel pre-tokenizer, byte b at id b + 3."""
    # the GPT-2 byte-to-character table: printable bytes map to themselves, the rest to 256+n
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2}
    for b in range(256):
        vocab[table[b]] = b + 3
    return {
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
        "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False},
        "post_processor": None,
        "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False},
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None,
                  "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False, "vocab": vocab, "merges": []},
    }
