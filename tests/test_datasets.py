"""Dataset preparation: tokenize text and conversations to flat token files, read them back,
pack documents into the microbatches a training step takes, and train on them."""
import json

import numpy as np

from shadowspill_b200.data.prepare import ByteTokenizer, TokenDataset, prepare


def _corpus(tmp_path, n=40):
    rng = np.random.default_rng(0)
    words = ["spill", "fetch", "evict", "plan", "stage", "tensor", "host", "link", "step", "update"]
    paths = []
    for i in range(n):
        p = tmp_path / f"doc{i}.txt"
        p.write_text(" ".join(rng.choice(words, size=int(rng.integers(10, 60)))))
        paths.append(str(p))
    return paths


def test_text_dataset_round_trip_and_packing(tmp_path):
    meta = prepare("text", _corpus(tmp_path), tmp_path / "out", "bytes", val_fraction=0.1, seed=3)
    assert meta["dtype"] == "uint16" and meta["train"]["documents"] == 36 and meta["val"]["documents"] == 4
    assert json.loads((tmp_path / "out" / "meta.json").read_text())["tokenizer"]["kind"] == "bytes"
    ds = TokenDataset(tmp_path / "out", "train")
    assert len(ds) == 36 and ds.mask is None
    ids, _ = ds.document(0)
    assert ids[-1] == ByteTokenizer.eos_id and "s" in ByteTokenizer().decode(ids)
    seen = 0
    for batch in ds.batches(tokens_per_step=2048, microbatch_tokens=1024, slots=9, seed=1):
        assert len(batch) == 2
        total_weight = 0.0
        for mb in batch:
            assert mb.tokens.shape == (1024,) and mb.cu_seqlens.shape == (10,) and mb.cu_seqlens[-1] == 1024
            assert (np.diff(mb.cu_seqlens) >= 0).all()
            carries = mb.targets >= 0
            assert (mb.weights[~carries] == 0).all()
            assert (mb.targets[carries] == mb.tokens[1:][carries[:-1]]).all()      # next-token targets
            total_weight += float(mb.weights.sum())
            seen += int((np.diff(mb.cu_seqlens) > 0).sum())
        assert abs(total_weight - 1.0) < 1e-5                                     # 1/N over the global batch
    assert seen >= 36                                                             # every document was served


def test_chat_dataset_masks_everything_but_assistant_tokens_and_trains(tmp_path):
    path = tmp_path / "chats.jsonl"
    rng = np.random.default_rng(1)
    with open(path, "w") as f:
        for i in range(30):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"question {i} " + "x" * int(rng.integers(5, 40))},
                                             {"role": "assistant", "content": f"answer {i % 3}"}]}) + "\n")
    meta = prepare("chat", [str(path)], tmp_path / "chat", "bytes", val_fraction=0.0)
    assert meta["train"]["documents"] == 30 and meta["val"]["documents"] == 0
    ds = TokenDataset(tmp_path / "chat")
    ids, mask = ds.document(0)
    text = ByteTokenizer().decode(ids[mask.astype(bool)])
    assert text.startswith("answer") and "question" not in text
    from shadowspill_b200.models.config import DecoderConfig
    from shadowspill_b200.planning.plan import SearchOptions
    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    cfg = DecoderConfig("llama3", 2, 64, 4, 2, 16, 128, ds.vocab_size)
    session = TrainingSession(TrainingSetup(model=cfg, device_gib=0.53, spill_gib=0.25, tokens_per_step=1024,
                                            microbatch_tokens=512, lr=1e-2, device="cpu", dtype="float32",
                                            profile=False, calibrate=False, slots=17,
                                            search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1)))
    losses = []
    for epoch in range(6):
        for batch in ds.batches(1024, 512, slots=session.slots, seed=epoch):
            losses.append(session.step(batch).loss)
    session.close()
    assert losses[-1] < 0.7 * losses[0], losses        # the three answers are learnable
