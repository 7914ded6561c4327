"""Encoder service on CPU ranks (gloo): wire format, producer / consumer streaming with prefetch, resume handshake,
a dropped message surfacing as a bounded timeout with fallback, and the full training entry with encoder ranks."""

import json
import os

import pytest
import torch

from dist_utils import run_distributed

EXAMPLE = os.path.join(os.path.dirname(__file__), "..", "examples", "hunyuanvideo")


def _spec():
    from teletron_b200.encoder_service import MessageSpec
    return MessageSpec.from_flags(9, (64, 32), max_text_len=8, text_dim=16, pooled_dim=4)


def test_message_round_trip_and_header_checks():
    from teletron_b200.encoder_service import ProtocolError, pack_message, unpack_message
    spec = _spec()
    g = torch.Generator().manual_seed(0)
    pe = torch.randn(5, 16, generator=g).bfloat16()
    ce = torch.randn(4, generator=g).bfloat16()
    lat = torch.randn(16, 3, 4, 8, generator=g).bfloat16()
    first = torch.randn(16, 1, 4, 8, generator=g).bfloat16()
    msg = pack_message(spec, 70000, pe, ce, first, lat)
    assert msg.numel() == spec.numel and spec.nbytes == 2 * spec.numel
    out = unpack_message(spec, msg, expect_seq=70000)
    assert out["text_len"] == 5 and out["prompt_attention_mask"].sum() == 5
    assert torch.equal(out["prompt_embeds"][0, :5], pe) and out["prompt_embeds"][0, 5:].abs().sum() == 0
    assert torch.equal(out["latents"][0], lat) and torch.equal(out["first_frame_latents"][0], first)
    with pytest.raises(ProtocolError):
        unpack_message(spec, msg, expect_seq=70001)
    bad = msg.clone()
    bad[0] = 0
    with pytest.raises(ProtocolError):
        unpack_message(spec, bad)
    with pytest.raises(ProtocolError):
        pack_message(spec, 0, torch.zeros(9, 16).bfloat16(), ce, first, lat)


def _stream(rank, world, n_items, start_iter, drop_seq):
    """rank 0: consumer; rank 1: producer serving it."""
    from teletron_b200.encoder_service import EncoderConsumer, EncoderTimeout, pack_message, producer_loop
    from teletron_b200.parallel.state import CommPair
    import torch.distributed as dist
    spec = _spec()
    pair = CommPair(producer=1, consumer=0, dp_rank=0, dp_size=1)

    def sample(seq):
        g = torch.Generator().manual_seed(seq)
        return (torch.randn(3 + seq % 4, 16, generator=g).bfloat16(), torch.randn(4, generator=g).bfloat16(),
                torch.randn(16, 1, 4, 8, generator=g).bfloat16(), torch.randn(16, 3, 4, 8, generator=g).bfloat16())
    if rank == 1:
        t = torch.zeros(1, dtype=torch.int64)
        dist.irecv(t, src=0).wait()
        start = int(t)
        it = iter(range(start, start + n_items))
        sent = producer_loop([pair], {0: it}, lambda s, seq: pack_message(spec, seq, *sample(seq)), {0: start},
                             max_items=n_items, drop=(lambda c, s: s == drop_seq) if drop_seq is not None else None)
        return ("producer", start, sent[0])
    fallback_used = []

    def fallback():
        fallback_used.append(True)
        return {"latents": torch.zeros(1, 16, 3, 4, 8)}
    cons = EncoderConsumer(pair, None, device=torch.device("cpu"), spec=spec, timeout=2.0,
                           fallback=fallback if drop_seq is not None else None)
    cons.handshake(start_iter, num_messages=n_items if drop_seq is None else n_items - 1)
    got = []
    n_expected = n_items if drop_seq is None else n_items - 1
    for i in range(n_expected):
        b = cons.next_batch()
        got.append(b)
        if fallback_used:
            # drain what the producer still sends so that both sides leave with nothing in flight
            buf = torch.empty(spec.numel, dtype=torch.bfloat16)
            for _ in range(n_expected - i - 1):
                dist.recv(buf, src=1)
            break
        seq = start_iter + i
        pe, ce, first, lat = sample(seq)
        assert torch.equal(b["latents"][0], lat) and torch.equal(b["clip_text_embed"][0], ce)
        assert int(b["prompt_attention_mask"].sum()) == pe.shape[0]
    cons.close()
    return ("consumer", len(got), bool(fallback_used), cons.bytes_received)


def test_stream_with_prefetch_and_resume():
    res = run_distributed(_stream, 2, 6, 40, None)
    assert res[1] == ("producer", 40, 6)
    assert res[0][:3] == ("consumer", 6, False) and res[0][3] == 6 * _spec().nbytes


def test_dropped_message_is_detected_and_falls_back():
    # message 41 is encoded but never sent: the consumer sees sequence 42 where it expects 41 (or times out) and
    # switches to its fallback source instead of hanging
    res = run_distributed(_stream, 2, 4, 40, 41)
    assert res[0][2] is True


def _two_producers(rank, world, n_items, start_iter):
    """rank 0: consumer fed by ranks 1 and 2 in turn (more encoder ranks than DiT groups)."""
    from teletron_b200.encoder_service import EncoderConsumer, pack_message, producer_loop
    from teletron_b200.parallel.state import build_comm_pairs
    import torch.distributed as dist
    spec = _spec()
    pairs = build_comm_pairs(1, 2, 1, 1)
    assert [(p.producer, p.lane, p.lanes) for p in pairs] == [(1, 0, 2), (2, 1, 2)]

    def sample(seq):
        g = torch.Generator().manual_seed(seq)
        return (torch.randn(3 + seq % 4, 16, generator=g).bfloat16(), torch.randn(4, generator=g).bfloat16(),
                torch.randn(16, 1, 4, 8, generator=g).bfloat16(), torch.randn(16, 3, 4, 8, generator=g).bfloat16())
    if rank > 0:
        mine = [p for p in pairs if p.producer == rank]
        t = torch.zeros(1, dtype=torch.int64)
        dist.irecv(t, src=0).wait()
        start = int(t)
        lane, lanes = mine[0].lane, mine[0].lanes
        q0 = start + ((lane - start) % lanes)
        items = range(q0, start + n_items, lanes)          # this lane's sequence numbers
        sent = producer_loop(mine, {0: iter(items)}, lambda s, seq: pack_message(spec, seq, *sample(seq)), {0: q0},
                             max_items=len(items))
        return sent[0]
    cons = EncoderConsumer(pairs, None, device=torch.device("cpu"), spec=spec, timeout=20.0)
    cons.handshake(start_iter, num_messages=n_items)
    for i in range(n_items):
        b = cons.next_batch()
        assert torch.equal(b["latents"][0], sample(start_iter + i)[3]), i
    cons.close()
    return cons.bytes_received


def test_two_encoder_ranks_feed_one_consumer_in_turn():
    res = run_distributed(_two_producers, 3, 7, 41)
    # sequence numbers 41 .. 47: the odd ones (lane 1) come from rank 2, the even ones from rank 1
    assert res[0] == 7 * _spec().nbytes and res[1] == 3 and res[2] == 4


def _train_with_encoder_rank(rank, world, tmp, enc=1):
    import importlib
    import sys
    sys.path.insert(0, EXAMPLE)
    import pretrain_hunyuanvideo as entry
    importlib.reload(entry)
    from teletron_b200.training import pretrain
    os.environ["TELETRON_B200_KEEP_PG"] = "1"
    log = os.path.join(tmp, "log.jsonl")
    argv = ["--model-size", "tiny", "--dataset-type", "FakeDataset", "--num-frames", "9", "--video-resolution", "64", "64",
            "--text-len", "16", "--train-iters", "3", "--lr", "1e-4", "--use-distributed-optimizer", "--num-workers", "0",
            "--context-parallel-size", "2", "--distributed-vae", "--distributed-vae-world-size", str(enc),
            "--encoder-preset", "tiny", "--encoder-max-text-len", "16", "--jsonl-log", log, "--distributed-timeout-minutes", "2"]
    model = pretrain(entry.train_valid_test_datasets_provider, entry.model_provider, entry.forward_step,
                     producer_process=entry.producer_process, extra_args_provider=entry.extra_args_provider, argv=argv)
    return "dit" if model is not None else "encoder"


def test_training_entry_with_one_encoder_rank(tmp_path):
    """3 CPU ranks: 2 DiT ranks (cp = 2) + 1 encoder rank running the tiny VAE / LLaMA / CLIP and streaming samples."""
    res = run_distributed(_train_with_encoder_rank, 3, str(tmp_path), timeout=420)
    assert res == ["dit", "dit", "encoder"]
    lines = [json.loads(l) for l in open(tmp_path / "log.jsonl")]
    assert len(lines) == 3 and all(l["loss"] == l["loss"] for l in lines)


def test_training_entry_with_two_encoder_ranks_for_one_dit_group(tmp_path):
    """4 CPU ranks: 2 DiT ranks (cp = 2, one data-parallel replica) fed by 2 encoder ranks in turn."""
    res = run_distributed(_train_with_encoder_rank, 4, str(tmp_path), 2, timeout=420)
    assert res == ["dit", "dit", "encoder", "encoder"]
    lines = [json.loads(l) for l in open(tmp_path / "log.jsonl")]
    assert len(lines) == 3 and all(l["loss"] == l["loss"] for l in lines)
