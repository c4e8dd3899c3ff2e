"""Prepare tokenized datasets: text for next-token pretraining, conversations for fine-tuning.

    python -m shadowspill_b200.data.prepare text  --input corpus/*.txt --output data/corpus --tokenizer bytes
    python -m shadowspill_b200.data.prepare chat  --input chats.jsonl  --output data/chat   --tokenizer DIR

``text`` tokenizes documents (one per file, or one per line with ``--lines``), appends an
end-of-document token to each, and writes ``train.bin`` / ``val.bin`` (flat uint16 or uint32 token
ids) with ``train.idx`` / ``val.idx`` (int64 document offsets) and ``meta.json`` (tokenizer identity,
vocabulary size, counts). ``chat`` renders ``{"messages": [{"role", "content"}, ...]}`` records with
a chat template and writes, beside the tokens, a ``*.mask`` file (uint8) that is 1 on assistant
tokens: the positions that carry loss in fine-tuning.

Tokenizers: ``bytes`` (UTF-8 bytes + 2 special ids; no files needed) or a directory readable by
``transformers.AutoTokenizer.from_pretrained(..., local_files_only=True)`` (its chat template is
used when it has one). Nothing is downloaded.

``TokenDataset`` reads the files back (memory-mapped) and ``batches`` packs whole documents into
microbatches of fixed capacity: the ``HostMicrobatch`` lists ``TrainingSession.step`` and the
client's ``text_batch`` take.

Reference: tools/datasets (prepare_text.py, prepare_chat.py, tokenizer.py, corpus.py: ``train.bin``,
``val.bin`` and ``meta.json`` with the tokenizer's identity).
"""
from __future__ import annotations

import argparse
import glob
import hashlib
import json
import sys
from pathlib import Path
from typing import Iterable, Iterator

import numpy as np

from .synthetic import HostMicrobatch, pack_first_fit


class ByteTokenizer:
    """UTF-8 bytes as ids 0..255, end of document 256, role separator 257."""
    name = "bytes"
    vocab_size = 258
    eos_id = 256
    sep_id = 257

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")

    def identity(self) -> dict:
        return {"kind": "bytes", "vocab_size": self.vocab_size, "eos_id": self.eos_id}

    def render_chat(self, messages: list[dict]) -> tuple[list[int], list[int]]:
        """``<role>\\n<content><sep>`` per message; the mask covers assistant content and its separator."""
        ids, mask = [], []
        for m in messages:
            head = self.encode(m["role"] + "\n")
            body = self.encode(m["content"]) + [self.sep_id]
            ids += head + body
            mask += [0] * len(head) + [1 if m["role"] == "assistant" else 0] * len(body)
        return ids + [self.eos_id], mask + [0]


class PretrainedTokenizer:
    """A tokenizer directory on disk, through ``transformers`` (never the network)."""

    def __init__(self, directory: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(directory, local_files_only=True)
        self.name = str(directory)
        self.vocab_size = len(self.tok)
        self.eos_id = self.tok.eos_token_id if self.tok.eos_token_id is not None else self.vocab_size - 1
        files = sorted(p for p in Path(directory).iterdir() if p.is_file() and p.suffix in (".json", ".model", ".txt"))
        h = hashlib.sha256()
        for p in files:
            h.update(p.name.encode())
            h.update(p.read_bytes())
        self._digest = h.hexdigest()

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids))

    def identity(self) -> dict:
        return {"kind": "pretrained", "directory": self.name, "vocab_size": self.vocab_size,
                "eos_id": self.eos_id, "files_sha256": self._digest}

    def render_chat(self, messages: list[dict]) -> tuple[list[int], list[int]]:
        """With the tokenizer's own chat template: the mask marks what each assistant turn adds
        to the rendering of the conversation before it."""
        ids: list[int] = []
        mask: list[int] = []
        for i, m in enumerate(messages):
            upto = self.tok.apply_chat_template(messages[:i + 1], tokenize=True, add_generation_prompt=False)
            upto = list(upto["input_ids"] if isinstance(upto, dict) else upto)
            new = upto[len(ids):]
            mask += [1 if m["role"] == "assistant" else 0] * len(new)
            ids = upto
        return ids, mask


def load_tokenizer(spec: str):
    return ByteTokenizer() if spec == "bytes" else PretrainedTokenizer(spec)


# ------------------------------------------------------------------------ writing
def _documents(paths: list[str], lines: bool) -> Iterator[str]:
    for p in paths:
        text = Path(p).read_text(encoding="utf-8", errors="replace")
        if lines:
            yield from (ln for ln in text.splitlines() if ln.strip())
        else:
            yield text


def _write_split(out: Path, name: str, docs: list[np.ndarray], masks: list[np.ndarray] | None, dtype) -> dict:
    offsets = np.zeros(len(docs) + 1, dtype=np.int64)
    for i, d in enumerate(docs):
        offsets[i + 1] = offsets[i] + len(d)
    flat = np.concatenate(docs).astype(dtype) if docs else np.zeros(0, dtype=dtype)
    flat.tofile(out / f"{name}.bin")
    offsets.tofile(out / f"{name}.idx")
    if masks is not None:
        (np.concatenate(masks).astype(np.uint8) if masks else np.zeros(0, np.uint8)).tofile(out / f"{name}.mask")
    return {"documents": len(docs), "tokens": int(offsets[-1])}


def prepare(kind: str, inputs: list[str], output: str | Path, tokenizer="bytes", val_fraction: float = 0.01,
            lines: bool = False, seed: int = 0, max_tokens_per_document: int = 0) -> dict:
    """Tokenizes ``inputs`` into ``output``; returns the metadata also written to ``meta.json``."""
    tok = load_tokenizer(tokenizer) if isinstance(tokenizer, str) else tokenizer
    out = Path(output)
    out.mkdir(parents=True, exist_ok=True)
    docs: list[np.ndarray] = []
    masks: list[np.ndarray] | None = [] if kind == "chat" else None
    if kind == "text":
        for text in _documents(inputs, lines):
            ids = tok.encode(text) + [tok.eos_id]
            if max_tokens_per_document:
                ids = ids[:max_tokens_per_document]
            if len(ids) >= 2:
                docs.append(np.asarray(ids, dtype=np.int64))
    elif kind == "chat":
        for p in inputs:
            for ln in Path(p).read_text(encoding="utf-8").splitlines():
                if not ln.strip():
                    continue
                rec = json.loads(ln)
                ids, mask = tok.render_chat(rec["messages"])
                if max_tokens_per_document:
                    ids, mask = ids[:max_tokens_per_document], mask[:max_tokens_per_document]
                if len(ids) >= 2 and any(mask):
                    docs.append(np.asarray(ids, dtype=np.int64))
                    masks.append(np.asarray(mask, dtype=np.uint8))
    else:
        raise ValueError(f"unknown dataset kind {kind!r} (text | chat)")
    if not docs:
        raise ValueError("no documents with at least two tokens in the inputs")
    order = np.random.default_rng(seed).permutation(len(docs))
    n_val = min(len(docs) - 1, max(1 if val_fraction > 0 and len(docs) > 1 else 0, int(len(docs) * val_fraction)))
    val_ix, train_ix = sorted(order[:n_val].tolist()), sorted(order[n_val:].tolist())
    dtype = np.uint16 if tok.vocab_size <= 65536 else np.uint32
    meta = {"format": "ss-b200.tokens", "version": 1, "kind": kind, "dtype": np.dtype(dtype).name,
            "tokenizer": tok.identity(), "seed": seed,
            "train": _write_split(out, "train", [docs[i] for i in train_ix],
                                  None if masks is None else [masks[i] for i in train_ix], dtype),
            "val": _write_split(out, "val", [docs[i] for i in val_ix],
                                None if masks is None else [masks[i] for i in val_ix], dtype)}
    (out / "meta.json").write_text(json.dumps(meta, indent=1))
    return meta


# ------------------------------------------------------------------------ reading
class TokenDataset:
    """One split of a prepared dataset, memory-mapped."""

    def __init__(self, directory: str | Path, split: str = "train"):
        d = Path(directory)
        self.meta = json.loads((d / "meta.json").read_text())
        if self.meta.get("format") != "ss-b200.tokens":
            raise ValueError(f"{d} is not a prepared token dataset")
        self.tokens = np.memmap(d / f"{split}.bin", dtype=self.meta["dtype"], mode="r")
        self.offsets = np.fromfile(d / f"{split}.idx", dtype=np.int64)
        mask = d / f"{split}.mask"
        self.mask = np.memmap(mask, dtype=np.uint8, mode="r") if mask.exists() and mask.stat().st_size else None
        self.vocab_size = int(self.meta["tokenizer"]["vocab_size"])

    def __len__(self) -> int:
        return len(self.offsets) - 1

    def document(self, i: int) -> tuple[np.ndarray, np.ndarray | None]:
        a, b = int(self.offsets[i]), int(self.offsets[i + 1])
        return np.asarray(self.tokens[a:b], dtype=np.int64), (None if self.mask is None else np.asarray(self.mask[a:b]))

    def batches(self, tokens_per_step: int, microbatch_tokens: int, slots: int, seed: int = 0,
                max_len: int | None = None) -> Iterator[list[HostMicrobatch]]:
        """Global batches of whole documents (longer ones are cut at ``max_len``), packed first-fit
        into ``tokens_per_step // microbatch_tokens`` microbatches; loss weights are 1/N over the
        positions that carry loss in the global batch (every next-token position for text, the
        assistant tokens for chat)."""
        n_mb = tokens_per_step // microbatch_tokens
        max_len = min(max_len or microbatch_tokens, microbatch_tokens)
        order = np.random.default_rng(seed).permutation(len(self))
        cursor = 0
        while cursor < len(order):
            docs, total = [], 0
            while cursor < len(order) and len(docs) < n_mb * (slots - 1):
                ids, mask = self.document(int(order[cursor]))
                ids, mask = ids[:max_len], (None if mask is None else mask[:max_len])
                if total + len(ids) > tokens_per_step:
                    break
                docs.append((ids, mask))
                total += len(ids)
                cursor += 1
            if not docs:
                cursor += 1                      # a document that cannot fit anywhere is skipped
                continue
            try:
                bins = pack_first_fit([len(d[0]) for d in docs], microbatch_tokens, n_mb)
            except ValueError:
                docs = docs[:-1]                 # fragmentation: carry the last document over
                cursor -= 1
                if not docs:
                    cursor += 1
                    continue
                bins = pack_first_fit([len(d[0]) for d in docs], microbatch_tokens, n_mb)
            yield _microbatches(docs, bins, microbatch_tokens, slots)


def _microbatches(docs, bins, T: int, slots: int) -> list[HostMicrobatch]:
    out, counted = [], 0
    for members in bins:
        members = members[:slots - 1]
        tokens = np.zeros(T, dtype=np.int64)
        targets = np.full(T, -1, dtype=np.int64)
        weights = np.zeros(T, dtype=np.float32)
        positions = np.zeros(T, dtype=np.int32)
        cu, pos, longest = [0], 0, 1
        for i in members:
            ids, mask = docs[i]
            n = len(ids)
            tokens[pos:pos + n] = ids
            positions[pos:pos + n] = np.arange(n, dtype=np.int32)
            targets[pos:pos + n - 1] = ids[1:]
            carries = np.ones(n - 1, dtype=bool) if mask is None else mask[1:].astype(bool)
            targets[pos:pos + n - 1][~carries] = -1
            weights[pos:pos + n - 1][carries] = 1.0
            counted += int(carries.sum())
            pos += n
            cu.append(pos)
            longest = max(longest, n)
        if pos < T:                              # padding forms its own sequence without loss
            positions[pos:] = np.arange(T - pos, dtype=np.int32)
            longest = max(longest, T - pos)
            cu.append(T)
        cu += [T] * (slots + 1 - len(cu))
        out.append(HostMicrobatch(tokens, targets, weights, positions, np.asarray(cu, dtype=np.int32), longest))
    for mb in out:
        mb.weights /= max(counted, 1)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("kind", choices=["text", "chat"])
    ap.add_argument("--input", nargs="+", required=True, help="files or glob patterns")
    ap.add_argument("--output", required=True)
    ap.add_argument("--tokenizer", default="bytes", help="'bytes' or a tokenizer directory on disk")
    ap.add_argument("--val-fraction", type=float, default=0.01)
    ap.add_argument("--lines", action="store_true", help="text: one document per non-empty line")
    ap.add_argument("--max-tokens-per-document", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    paths = sorted({p for pat in a.input for p in (glob.glob(pat) or [pat])})
    meta = prepare(a.kind, paths, a.output, a.tokenizer, a.val_fraction, a.lines, a.seed,
                   a.max_tokens_per_document)
    print(json.dumps({k: meta[k] for k in ("kind", "dtype", "tokenizer", "train", "val")}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
