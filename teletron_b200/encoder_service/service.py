"""Distributed multimodal-encoder service: producer ranks and their DiT-side consumers.

Dedicated ranks at the tail of the world run the VAE and the two text encoders and stream one
flat message per sample to the first rank of each TP x CP block over ``torch.distributed`` p2p
(NCCL on GPU), as in ``teletron/models/hunyuanvideo/producer.py:105-236`` and
``teletron/training/utils.py:84-174``.  What differs:

* the consumer keeps one ``irecv`` posted *ahead* of the step that needs it, so the transfer runs
  under DiT compute instead of blocking at the top of the step (``utils.py:115-116``);
* the receive buffer is sized from the flags (the reference pulls a full sample from a local
  dataloader just to read its shape, ``utils.py:98-110``);
* messages carry a checked header (:mod:`.protocol`), waits are bounded and raise
  :class:`EncoderTimeout`, and a consumer that loses its producer can fall back to a local sample
  source instead of hanging until the process-group timeout;
* producers use their own device (``LOCAL_RANK``), not ``cuda:{rank - dit_world}`` which aliases
  DiT GPUs on one node (``producer.py:113-115``).
"""

from __future__ import annotations

import collections
import threading
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..parallel import state as ps
from ..parallel.state import CommPair
from .protocol import MessageSpec, ProtocolError, pack_message, unpack_message

QUEUE_DEPTH = 2            # encoded samples buffered per consumer (producer.py:24-26)
MAX_OUTSTANDING_SENDS = 1


class EncoderTimeout(RuntimeError):
    pass


class _Request:
    """A p2p request whose completion can be polled on every backend.

    NCCL requests answer ``is_completed()`` from a CUDA event.  Gloo requests only make progress inside ``wait()``,
    and a ``wait(timeout)`` that runs out tears the connection down, so there a helper thread sits in ``wait()`` and
    sets an event (the CPU path is for tests and small jobs; one short-lived thread per message is acceptable)."""

    def __init__(self, req):
        self._req = req
        self._event = None
        self._error = None
        if dist.get_backend() != "nccl":
            self._event = threading.Event()
            threading.Thread(target=self._run, daemon=True).start()

    def _run(self):
        try:
            self._req.wait()
        except Exception as e:          # a closed connection: reported to whoever waits
            self._error = e
        self._event.set()

    def done(self) -> bool:
        if self._event is not None:
            return self._event.is_set()
        return self._req.is_completed()

    def wait(self, timeout: Optional[float], what: str) -> None:
        """Bounded wait: a lost peer surfaces as :class:`EncoderTimeout` instead of a hang."""
        if self._event is not None:
            if not self._event.wait(timeout if timeout and timeout > 0 else None):
                raise EncoderTimeout(f"timed out after {timeout:.1f}s waiting for {what}")
            if self._error is not None:
                raise EncoderTimeout(f"{what}: {self._error}")
            return
        if timeout and timeout > 0:
            t0 = time.monotonic()
            while not self._req.is_completed():
                if time.monotonic() - t0 > timeout:
                    raise EncoderTimeout(f"timed out after {timeout:.1f}s waiting for {what}")
                time.sleep(0.001)
        self._req.wait()


class Encoders:
    """The three encoders a producer runs.  Each is a callable so tests can plug in stand-ins.

    ``vae(pixels [B, 3, F, H, W]) -> latents [B, 16, f, h, w]`` (already scaled),
    ``text(prompts: List[str]) -> (embeds [B, L, 4096], mask [B, L])``, ``clip(prompts) -> [B, 768]``.
    """

    def __init__(self, vae: Callable, text: Callable, clip: Callable):
        self.vae, self.text, self.clip = vae, text, clip

    @staticmethod
    def build_default(device, dtype=torch.bfloat16, vae_tiling: bool = True, max_text_len: int = 256,
                      preset: str = "default", text_dim: int = 4096, pooled_dim: int = 768) -> "Encoders":
        """The real encoders (random weights unless paths are configured): a 32-layer LLaMA-style decoder, CLIP-L text
        and the 3-D causal VAE; ``preset="tiny"`` shrinks all three for CPU tests."""
        from ..models.vae import AutoencoderKLHunyuanVideo
        from ..models.text_encoders import ClipTextEncoder, LlamaTextEncoder, clip_text_config, llama_config
        if preset == "tiny":
            vae = AutoencoderKLHunyuanVideo(block_out_channels=(32, 32, 32, 32)).to(device, dtype).eval()
            llama = LlamaTextEncoder(max_length=max_text_len, device=device, dtype=dtype,
                                     config=llama_config(2, text_dim, 4, 2, 2 * text_dim, 1000))
            clip = ClipTextEncoder(device=device, dtype=dtype, max_length=16, config=clip_text_config(2, pooled_dim, 4, 500, 16))
        else:
            vae = AutoencoderKLHunyuanVideo().to(device, dtype).eval()
            llama = LlamaTextEncoder(max_length=max_text_len, device=device, dtype=dtype)
            clip = ClipTextEncoder(device=device, dtype=dtype)
        vae.enable_tiling(vae_tiling)
        sf = 0.476986

        @torch.no_grad()
        def vae_fn(pixels):
            return vae.encode(pixels.to(device, dtype)) * sf
        return Encoders(vae_fn, llama, clip)


def encode_sample(sample: Dict, enc: Encoders, spec: MessageSpec, seq: int, device) -> torch.Tensor:
    """Dataset item (or collated batch of 1) -> packed message on ``device``."""
    images = sample["images"]
    if images.dim() == 4:
        images = images[None]
    pixels = images.permute(0, 2, 1, 3, 4)                                  # [B, 3, F, H, W]
    latents = enc.vae(pixels)
    first = sample.get("first_ref_image")
    if first is None:
        first_px = pixels[:, :, :1]
    else:
        first = first if first.dim() == 4 else first[None]                   # [B, 3, H, W]
        first_px = first[:, :, None]
    first_lat = enc.vae(first_px)
    prompt = sample["prompt"]
    prompts = list(prompt) if isinstance(prompt, (list, tuple)) else [prompt]
    embeds, mask = enc.text(prompts)
    L = int(mask[0].sum())
    pooled = enc.clip(prompts)
    return pack_message(spec, seq, embeds[0, :L].to(device, torch.bfloat16), pooled[0].to(device, torch.bfloat16),
                        first_lat[0].to(device, torch.bfloat16), latents[0].to(device, torch.bfloat16))


def spec_from_args(args) -> MessageSpec:
    return MessageSpec.from_flags(args.num_frames, args.video_resolution, args.encoder_max_text_len,
                                  args.encoder_text_dim, args.encoder_pooled_dim)


def producer_loop(pairs: List[CommPair], iterators: Dict[int, object], encode: Callable[[Dict, int], torch.Tensor],
                  start_seq: Dict[int, int], max_items: Optional[int] = None, idle_sleep: float = 0.002,
                  drop: Optional[Callable[[int, int], bool]] = None, stall_timeout: Optional[float] = None) -> Dict[int, int]:
    """Round-robin service of all consumers: keep up to ``QUEUE_DEPTH`` encoded samples per consumer and
    one outstanding ``isend`` each.  ``iterators[c]`` yields the samples of this producer's lane only and
    ``start_seq[c]`` is the lane's first sequence number; consecutive items are ``lanes`` sequence numbers apart.
    ``drop(consumer, seq)`` is a host-side fault-injection hook for the
    tests (a message that is encoded but never sent).  A consumer whose receive does not match a send within
    ``stall_timeout`` seconds is taken for lost and no longer served, so one dead DiT block cannot starve the
    others.  Returns the number of messages sent per consumer."""
    queues = {p.consumer: collections.deque() for p in pairs}
    inflight = {p.consumer: collections.deque() for p in pairs}
    seq = dict(start_seq)
    sent = {p.consumer: 0 for p in pairs}
    produced = {p.consumer: 0 for p in pairs}
    exhausted = set()
    lost = set()
    while True:
        progress = False
        for p in pairs:
            c = p.consumer
            if c in lost:
                continue
            if stall_timeout and inflight[c] and time.monotonic() - inflight[c][0][2] > stall_timeout:
                lost.add(c)
                queues[c].clear()
                inflight[c].clear()
                continue
            while inflight[c] and inflight[c][0][0].done():
                inflight[c].popleft()
                progress = True
            if c not in exhausted and len(queues[c]) < QUEUE_DEPTH and (max_items is None or produced[c] < max_items):
                try:
                    sample = next(iterators[c])
                except StopIteration:
                    exhausted.add(c)
                    continue
                queues[c].append((seq[c], encode(sample, seq[c])))
                seq[c] += p.lanes                       # the consumer's other producers carry the sequence numbers in between
                produced[c] += 1
                progress = True
            if queues[c] and len(inflight[c]) < MAX_OUTSTANDING_SENDS:
                s, msg = queues[c].popleft()
                if drop is not None and drop(c, s):
                    continue
                inflight[c].append((_Request(dist.isend(msg, dst=c, group=p.group)), msg, time.monotonic()))
                sent[c] += 1
                progress = True
        done = all(c in lost or ((c in exhausted or (max_items is not None and produced[c] >= max_items))
                                 and not queues[c] and not inflight[c]) for c in queues)
        if done:
            return sent
        if not progress:
            time.sleep(idle_sleep)


def producer_process(args, train_valid_test_datasets_provider: Callable, encoders: Optional[Encoders] = None) -> None:
    """Body of an encoder rank (called from :func:`teletron_b200.training.pretrain`)."""
    from ..training.pretrain import build_train_valid_test_data_iterators
    device = args.device
    pairs = ps.get_producer_pairs()
    if not pairs:
        return
    spec = spec_from_args(args)
    enc = encoders or Encoders.build_default(device, args.params_dtype, vae_tiling=bool(args.vae_tiling),
                                             max_text_len=args.encoder_max_text_len, preset=args.encoder_preset,
                                             text_dim=args.encoder_text_dim, pooled_dim=args.encoder_pooled_dim)
    # handshake: every consumer tells us the iteration it resumes from (training.py:208-220, producer.py:137-153)
    start = {}
    reqs = []
    for p in pairs:
        t = torch.zeros(1, dtype=torch.int64, device=device)
        reqs.append((p, t, _Request(dist.irecv(t, src=p.consumer, group=p.group))))
    for p, t, r in reqs:
        r.wait(args.distributed_timeout_minutes * 60.0, f"handshake from consumer {p.consumer}")
        start[p.consumer] = int(t.item())
    iterators, first, count = {}, {}, 0
    for p in pairs:
        # Sample q of consumer d is dataset item q * dp + d.  A producer that carries lane l of L lanes serves
        # q = l, l + L, ... which is exactly the shard (rank l * dp + d of L * dp) of a data-parallel sampler, so the
        # samples of the other lanes are never materialised here.
        begin = start[p.consumer]
        q0 = begin + ((p.lane - begin) % p.lanes)
        end = max(begin, args.train_iters * args.num_microbatches)
        args.consumed_train_samples = (q0 - p.lane) // p.lanes * (p.lanes * p.dp_size) * args.micro_batch_size
        it, _, _ = build_train_valid_test_data_iterators(train_valid_test_datasets_provider, args,
                                                         dp_rank=p.lane * p.dp_size + p.dp_rank, dp_size=p.lanes * p.dp_size)
        iterators[p.consumer] = it
        first[p.consumer] = q0
        count = max(count, len(range(q0, end, p.lanes)))
    producer_loop(pairs, iterators, lambda s, q: encode_sample(s, enc, spec, q, device), first, max_items=count)


class _Lane:
    """Receive state of one producer feeding this consumer."""

    def __init__(self, pair: CommPair, numel: int, device):
        self.pair = pair
        self.bufs = [torch.empty(numel, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.slot = 0
        self.req = None
        self.to_post = None         # receives still to post (None = unbounded)


class EncoderConsumer:
    """DiT-side endpoint: double-buffered receive per producer, one message per producer always in flight ahead of use.

    ``pair`` is one :class:`CommPair` or the list of this rank's pairs (``parallel.state.get_consumer_pairs()``):
    with several producers, sample ``seq`` arrives from the producer whose lane is ``seq % lanes``."""

    def __init__(self, pair, args=None, device=None, spec: Optional[MessageSpec] = None,
                 timeout: Optional[float] = None, fallback: Optional[Callable[[], Dict]] = None):
        pairs = sorted(pair, key=lambda p: p.lane) if isinstance(pair, (list, tuple)) else [pair]
        if [p.lane for p in pairs] != list(range(len(pairs))) or any(p.lanes != len(pairs) for p in pairs):
            raise ValueError("the consumer's pairs must cover lanes 0 .. lanes-1 exactly once")
        self.pair = pairs[0]
        self.device = device
        self.spec = spec or spec_from_args(args)
        self.timeout = timeout if timeout is not None else (args.distributed_timeout_minutes * 60.0 if args else None)
        self.fallback = fallback
        self._lanes = [_Lane(p, self.spec.numel, device) for p in pairs]
        self._seq = 0
        self._args = args
        self.bytes_received = 0

    def handshake(self, iteration: int, num_messages: Optional[int] = None) -> None:
        """Tell every producer where to resume; ``num_messages`` bounds how many receives will ever be posted."""
        t = torch.tensor([iteration], dtype=torch.int64, device=self.device)
        for lane in self._lanes:
            dist.isend(t, dst=lane.pair.producer, group=lane.pair.group).wait()
        self._seq = iteration
        if num_messages is None and self._args is not None:
            # never leave an unmatched receive behind at shutdown
            num_messages = max(0, self._args.train_iters - iteration) * self._args.num_microbatches
        n = len(self._lanes)
        for i, lane in enumerate(self._lanes):
            if num_messages is not None:
                lane.to_post = sum(1 for q in range(iteration, iteration + num_messages) if q % n == i)
            self._post(lane)

    def _post(self, lane: _Lane) -> None:
        if lane.to_post is not None:
            if lane.to_post <= 0:
                lane.req = None
                return
            lane.to_post -= 1
        lane.req = _Request(dist.irecv(lane.bufs[lane.slot], src=lane.pair.producer, group=lane.pair.group))

    def next_batch(self) -> Dict[str, torch.Tensor]:
        """The sample for this step; immediately re-posts the receive for that producer's next one."""
        lane = self._lanes[self._seq % len(self._lanes)]
        if lane.req is None:
            self._post(lane)
        if lane.req is None:
            raise RuntimeError("the encoder stream is exhausted (all scheduled samples were received)")
        try:
            lane.req.wait(self.timeout, f"sample {self._seq} from encoder rank {lane.pair.producer}")
            out = unpack_message(self.spec, lane.bufs[lane.slot], expect_seq=self._seq)
        except (EncoderTimeout, ProtocolError):
            if self.fallback is None:
                raise
            lane.req = None
            self._seq += 1
            return self.fallback()
        self.bytes_received += self.spec.nbytes
        self._seq += 1
        lane.slot ^= 1
        self._post(lane)                  # prefetch: lands while this step computes
        out.pop("seq")
        out.pop("text_len")
        return out

    def close(self):
        for lane in self._lanes:
            lane.req = None
