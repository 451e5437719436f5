"""Data package on CPU: tokenizers, text packing + resume, chat validation / label masking / packing, processors,
the DSV4 encoder driven by a stand-in encoding module.

Models the reference's tests/unit_tests/patches/test_chat_dataset*.py, test_dsv4_encoder.py and
tests/unit_tests/hf_datasets/test_chat_processors.py.
"""

import json
import textwrap

import pytest
import torch

from titan_b200.data.chat_dataset import ChatDataLoader, labels_for_token_ranges, validate_messages
from titan_b200.data.chat_encoders import ChatMLEncoder, DSV4ChatEncoder, chatml_assistant_ranges
from titan_b200.data.chat_processors import (
    import_chat_processor,
    process_gsm8k_sample,
    process_tau_sample,
    process_wordle_sample,
    process_yelp_sample,
)
from titan_b200.data.text_datasets import TextDataLoader
from titan_b200.data.tokenizer import ByteTokenizer, build_tokenizer, render_chatml


def test_byte_tokenizer_roundtrip_and_specials():
    tok = ByteTokenizer()
    ids = tok.encode("hé<|im_start|>x", add_bos=True, add_eos=True)
    assert ids[0] == tok.bos_id and ids[-1] == tok.eos_id and 259 in ids
    assert tok.decode(ids[1:-1]) == "hé<|im_start|>x"
    assert build_tokenizer("byte").vocab_size == 261
    with pytest.raises(FileNotFoundError):
        build_tokenizer("/nonexistent/assets")


def test_hf_tokenizer_from_json_assets(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers

    vocab = {"<s>": 0, "</s>": 1, "hello": 2, "world": 3, "[UNK]": 4}
    t = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    t.pre_tokenizer = pre_tokenizers.Whitespace()
    t.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<s>", "eos_token": {"content": "</s>"}}))
    tok = build_tokenizer(str(tmp_path))
    assert tok.encode("hello world", add_bos=True, add_eos=True) == [0, 2, 3, 1]
    assert tok.bos_id == 0 and tok.eos_id == 1 and tok.vocab_size == 5


def test_text_loader_packs_and_resumes(tmp_path):
    docs = [{"text": "a" * n} for n in (30, 50, 20, 70, 40, 10, 90, 25)]
    f = tmp_path / "data.jsonl"
    f.write_text("\n".join(json.dumps(d) for d in docs))
    mk = lambda: TextDataLoader(dataset="c4_test", dataset_path=str(f), tokenizer=ByteTokenizer(), seq_len=32,  # noqa: E731
                                batch_size=2, dp_rank=0, dp_world_size=1, infinite=False, pin_memory=False)
    a = mk()
    it = iter(a)
    b1, l1 = next(it)
    assert b1["input"].shape == (2, 32) and torch.equal(b1["input"][:, 1:], l1[:, :-1])
    state = a.state_dict()
    b2, _ = next(it)
    r = mk()
    r.load_state_dict(state)
    rb2, _ = next(iter(r))
    assert torch.equal(b2["input"], rb2["input"])
    # the other data-parallel rank reads other documents
    o = TextDataLoader(dataset="c4_test", dataset_path=str(f), tokenizer=ByteTokenizer(), seq_len=32, batch_size=1,
                       dp_rank=1, dp_world_size=2, infinite=False, pin_memory=False)
    assert not torch.equal(next(iter(o))[0]["input"][0], b1["input"][0])
    with pytest.raises(ValueError, match="same data-parallel"):
        o.load_state_dict(state)


def test_enwiki_eod_and_alpaca_datasets_from_bundled_assets(monkeypatch):
    import os

    from titan_b200.data.text_datasets import _alpaca_text

    monkeypatch.chdir(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # default paths are repo-relative
    tok = ByteTokenizer()
    wiki = TextDataLoader(dataset="enwiki-eod", dataset_path=None, tokenizer=tok, seq_len=64, batch_size=2, dp_rank=0,
                          dp_world_size=1, infinite=False, pin_memory=False)
    batch, labels = next(iter(wiki))
    assert batch["input"].shape == (2, 64) and labels.shape == (2, 64)
    flat = torch.cat([batch["input"].reshape(-1), labels[:, -1:].reshape(-1)])
    assert tok.decode([t for t in flat.tolist() if t < 256]).startswith("A tensor core is a matrix")
    # every article ends with the end-of-document token before the next one starts
    first_article_len = 1 + len(   # BOS, then the text
        "A tensor core is a matrix multiply-accumulate unit inside a streaming multiprocessor. It multiplies small "
        "tiles of low-precision numbers and accumulates the products at higher precision.")
    stream = []
    for b, _ in TextDataLoader(dataset="enwiki-eod", dataset_path=None, tokenizer=tok, seq_len=64, batch_size=1,
                               dp_rank=0, dp_world_size=1, infinite=False, pin_memory=False):
        stream.extend(b["input"][0].tolist())
    assert stream[first_article_len] == tok.eos_id and stream[first_article_len + 1] == tok.bos_id

    alp = TextDataLoader(dataset="alpaca", dataset_path=None, tokenizer=tok, seq_len=48, batch_size=1, dp_rank=0,
                         dp_world_size=1, infinite=False, pin_memory=False)
    text = tok.decode([t for t in next(iter(alp))[0]["input"][0].tolist() if t < 256])
    assert text.startswith("Below is an instruction that describes a task.")
    assert "### Input:\ngood morning" in _alpaca_text({"instruction": "Translate.", "input": "good morning",
                                                        "output": "bonjour"})
    assert _alpaca_text({"text": "ready-made", "instruction": "ignored"}) == "ready-made"


def test_validate_messages_rules():
    ok = [{"role": "system", "content": "s"}, {"role": "user", "content": "u"},
          {"role": "assistant", "content": "", "tool_calls": [1]}, {"role": "tool", "content": "r1"},
          {"role": "tool", "content": "r2"}, {"role": "user", "content": "more"}, {"role": "assistant", "content": "a"}]
    validate_messages(ok)
    with pytest.raises(ValueError, match="at least 2"):
        validate_messages(ok[:1])
    with pytest.raises(ValueError, match="Unknown role"):
        validate_messages([{"role": "bot", "content": ""}, {"role": "assistant", "content": ""}])
    with pytest.raises(ValueError, match="First message must be 'user'"):
        validate_messages([{"role": "assistant", "content": ""}, {"role": "assistant", "content": ""}])
    with pytest.raises(ValueError, match="First message must be 'user' or 'system'"):
        validate_messages([{"role": "tool", "content": ""}, {"role": "user", "content": ""},
                           {"role": "assistant", "content": ""}])
    with pytest.raises(ValueError, match="Expected non-assistant"):
        validate_messages([{"role": "user", "content": ""}, {"role": "assistant", "content": ""},
                           {"role": "assistant", "content": ""}])


def test_label_masking_and_chatml_ranges():
    assert labels_for_token_ranges([11, 12, 13, 14, 15], [(2, 4)]) == [-100, 12, 13, -100, -100]
    tok = ByteTokenizer()
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
            {"role": "user", "content": "again"}, {"role": "assistant", "content": "ok"}]
    text, tokens, ranges = ChatMLEncoder().encode_messages_with_assistant_ranges(msgs, tok, tok.eos_id)
    assert text == render_chatml(msgs).rstrip("\n") and len(ranges) == 2
    for (s, e), reply in zip(ranges, ("yo", "ok")):
        assert tok.decode(tokens[s:e]).startswith(reply)
    assert chatml_assistant_ranges(tok, tok.encode("no header here"), tok.eos_id) == []


def test_chat_loader_packs_samples_with_restarting_positions():
    tok = ByteTokenizer()
    rows = [{"question": f"q{i}" * (i + 1), "answer": f"work{i} #### {i}"} for i in range(6)]
    dl = ChatDataLoader(tokenizer=tok, seq_len=160, batch_size=1, samples=rows, sample_processor=process_gsm8k_sample,
                        infinite=False, pin_memory=False)
    batch, labels = next(iter(dl))
    assert batch["input"].shape == (1, 160) and labels.shape == (1, 160)
    pos = batch["positions"][0]
    assert (pos == 0).sum() >= 2  # several samples share the row, each restarting at position 0
    sup = labels[0] != -100
    assert 0 < sup.sum() < 160
    # inside a sample a supervised label is the next input token
    inside = sup[:-1] & (pos[1:] != 0)
    assert torch.equal(labels[0][:-1][inside], batch["input"][0][1:][inside])
    # too-long samples are dropped, fully masked ones as well
    short = ChatDataLoader(tokenizer=tok, seq_len=16, batch_size=1, samples=rows, sample_processor=process_gsm8k_sample,
                           infinite=False, pin_memory=False)
    assert list(short) == [] and short.dropped_long == 6


def test_processors():
    g = process_gsm8k_sample({"question": "2+2?", "answer": "two and two #### 4"})
    assert g[1] == {"role": "assistant", "reasoning_content": "two and two", "content": "4"}
    t = process_tau_sample({"messages": json.dumps([{"role": "user", "content": "x"},
                                                    {"role": "assistant", "content": "y"}]),
                            "tools": json.dumps([{"name": "f"}])})
    assert t[0]["role"] == "system" and t[0]["tools"] == [{"name": "f"}]
    w = process_wordle_sample({"prompt": [{"role": "user", "content": ["a", "b"]}],
                               "completion": [{"role": "assistant", "content": "c"}]})
    assert w[0]["content"] == "a\nb" and w[1]["content"] == "c"
    with pytest.raises(KeyError):
        process_wordle_sample({"x": 1})
    assert process_yelp_sample({"text": " fine ", "label": 3})[1]["content"] == "4 stars"
    assert import_chat_processor("titan_b200.data.chat_processors:process_gsm8k_sample") is process_gsm8k_sample
    assert import_chat_processor("titan_b200.data.chat_processors.process_yelp_sample") is process_yelp_sample
    with pytest.raises(ValueError):
        import_chat_processor("nodots")


def test_dsv4_encoder_with_stand_in_encoding_module(tmp_path):
    mod = tmp_path / "encoding_dsv4.py"
    mod.write_text(textwrap.dedent('''
        def merge_tool_messages(messages):
            return list(messages)
        def sort_tool_results_by_call_order(messages):
            return list(messages)
        def _drop_thinking_messages(messages):
            return [{k: v for k, v in m.items() if k != "reasoning_content"} for m in messages]
        def render_message(idx, messages, thinking_mode="thinking", drop_thinking=True, reasoning_effort=None):
            m = messages[idx]
            think = m.get("reasoning_content")
            body = (f"<think>{think}</think>" if think and not drop_thinking else "") + (m.get("content") or "")
            return f"<{m['role']}>{body}</{m['role']}>\\n"
    '''))
    tok = ByteTokenizer()
    enc = DSV4ChatEncoder(str(mod), thinking_mode="thinking", drop_thinking=True)
    msgs = [{"role": "user", "content": "q"}, {"role": "assistant", "reasoning": "hmm", "content": "a"}]
    text, tokens, ranges = enc.encode_messages_with_assistant_ranges(msgs, tok, tok.eos_id)
    assert "<think>" not in text and tokens[-1] == tok.eos_id
    (s, e), = ranges
    assert tok.decode(tokens[s:e - 1]) == "<assistant>a</assistant>" and e == len(tokens)
    keep = DSV4ChatEncoder(str(mod), drop_thinking=False)
    assert "<think>hmm</think>" in keep.encode_messages_with_assistant_ranges(msgs, tok, tok.eos_id)[0]
    with pytest.raises(ValueError, match="thinking_mode"):
        DSV4ChatEncoder(str(mod), thinking_mode="deep")
    with pytest.raises(FileNotFoundError):
        DSV4ChatEncoder(str(tmp_path / "missing.py"))
