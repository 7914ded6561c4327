"""Encoder service ("distributed VAE"): producer ranks stream encoded samples to DiT ranks."""

from .protocol import MessageSpec, ProtocolError, pack_message, unpack_message  # noqa: F401
from .service import (EncoderConsumer, EncoderTimeout, Encoders, encode_sample, producer_loop,  # noqa: F401
                      producer_process)
