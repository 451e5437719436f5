"""DeepSeek-V4 packed streams (global TND): the layout derived from document positions, the packing of inputs / labels /
MTP pairs, and the model on a packed stream against the same documents run one by one.

Models what the reference covers in tests/unit_tests/models/test_deepseek_v4_tnd.py."""

from types import SimpleNamespace

import torch

from titan_b200.models.deepseek_v4 import DeepSeekV4Model, deepseekv4_configs
from titan_b200.models.deepseek_v4.tnd import build_packed_layout, compressed_block_starts, pack_global_tnd
from titan_b200.trainer.loss import IGNORE_INDEX


def _positions(*lengths):
    return torch.cat([torch.arange(n) for n in lengths])


def test_layout_of_three_documents():
    args = SimpleNamespace(compress_ratios=(1, 4), mtp_layer_compress_ratio=1)
    lay = build_packed_layout(_positions(5, 11, 8), args)
    assert lay.cu_seqlens_q.tolist() == [0, 5, 16, 24]
    assert lay.doc_ranges == ((0, 5), (5, 16), (16, 24))
    # complete blocks of 4: doc 0 has one (tokens 0-3), doc 1 two (5-8, 9-12), doc 2 two (16-19, 20-23)
    assert lay.block_starts_by_ratio[4].tolist() == [0, 5, 9, 16, 20]
    assert lay.cu_seqlens_cmp_kv[4].tolist() == [0, 1, 3, 5]
    assert lay.cmp_residual_k[4].tolist() == [1, 3, 0]
    assert lay.max_seqlen_q == 11 and lay.max_seqlen_cmp_kv[4] == 2 and lay.batch_size == 3 and lay.seq_len == 24


def test_block_needs_consecutive_positions_of_one_document():
    # a document of 6 tokens followed by one of 2: the block that would start at token 4 runs into the next document
    assert compressed_block_starts(_positions(6, 2), 4).tolist() == [0]


def test_packing_drops_padding_and_pairs_mtp_tokens_inside_documents():
    args = SimpleNamespace(compress_ratios=(1, 4), mtp_layer_compress_ratio=1, num_mtp_modules=1)
    # two rows of 8 main tokens + 1 MTP column; row 0 = docs of 3 and 5 tokens, row 1 = a doc of 6 then padding
    pos = torch.tensor([[0, 1, 2, 0, 1, 2, 3, 4, 5], [0, 1, 2, 3, 4, 5, -1, -1, -1]])
    inp = torch.arange(18).view(2, 9)
    lab = inp + 100
    x, y, extra = pack_global_tnd(inp, lab, pos, args)
    assert x.shape == (1, 14) and y.shape == (2, 1, 14) and extra["mtp_inputs"].shape == (1, 1, 14)
    assert x[0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14]
    assert extra["positions"][0].tolist() == [0, 1, 2, 0, 1, 2, 3, 4, 0, 1, 2, 3, 4, 5]
    assert extra["attention_masks"].doc_ranges == ((0, 3), (3, 8), (8, 14))
    main, mtp = y[0, 0].tolist(), y[1, 0].tolist()
    assert main == [100, 101, 102, 103, 104, 105, 106, 107, 109, 110, 111, 112, 113, 114]
    # the MTP label of a token is its successor's label unless the successor starts another document or is padding
    assert mtp[:3] == [101, 102, IGNORE_INDEX]
    assert mtp[3:8] == [104, 105, 106, 107, 108]  # token 7's successor (column 8) continues the document
    assert mtp[8:] == [110, 111, 112, 113, 114, IGNORE_INDEX]
    # where there is no valid successor the MTP input falls back to the token itself
    assert extra["mtp_inputs"][0, 0].tolist()[:3] == [1, 2, 2]


def test_model_on_packed_stream_matches_documents_run_alone():
    torch.manual_seed(0)
    cfg = deepseekv4_configs["smoketest"]()
    cfg.max_seq_len = 256
    cfg.num_mtp_modules = 1
    cfg.enable_indexer_loss = False
    cfg.index_topk = 64  # every visible block is selected: no near-tie in the top-k can flip between the two runs
    model = DeepSeekV4Model(cfg)
    model.init_states()
    model.eval()
    lens = (40, 150)  # neither a multiple of 4 nor of 128: both leave uncompressed tails
    total = sum(lens)
    tok = torch.randint(0, cfg.vocab_size, (1, total + 1))
    pos = torch.cat([_positions(*lens), torch.tensor([0])]).unsqueeze(0)
    x, y, extra = pack_global_tnd(tok, tok.clone(), pos, cfg)
    with torch.no_grad():
        packed = model(x, **extra)
        start = 0
        for n in lens:
            # oracle: the document alone, padded to a multiple of every ratio (causality keeps the padding from
            # reaching the first n positions; a block closed by padding is visible to padding queries only)
            pad = (-n) % 128
            doc = torch.cat([tok[:, start:start + n], torch.zeros(1, pad + 1, dtype=tok.dtype)], dim=1)
            alone = model(doc)
            torch.testing.assert_close(packed[0][:, start:start + n], alone[0][:, :n], atol=2e-4, rtol=1e-4)
            # MTP head: identical wherever the successor exists inside the document
            torch.testing.assert_close(packed[1][:, start:start + n - 1], alone[1][:, :n - 1], atol=2e-4, rtol=1e-4)
            start += n


def test_trainer_runs_packed_streams_on_two_ranks(tmp_path):
    from _launch import launch, losses

    log = launch(["--module", "deepseek_v4", "--config", "deepseek_v4_smoketest", "--comm.backend", "gloo",
                  "--training.steps", "2", "--job.dump_folder", str(tmp_path / "r"),
                  "--dataloader.documents_per_row", "3", "--model.overrides", '{"use_global_tnd": true}'], 2, 29790)
    assert "global TND: batch" in log
    ls = losses(log)
    assert len(ls) == 2 and all(0 < x < 20 for x in ls)
