"""A residual of several streams (hyper-connections): the connection part and the blocks that use it.

Instead of one residual row a token has ``streams`` of them, all equal to the embedding at the start, kept as
float32 [tokens, streams * hidden].  A sublayer f with its norm N is joined to them by three small tensors:

    u = sum_s in[s] X[s];   y = f(N(u));   X[t] <- sum_s mix[s, t] X[s] + out[t] * y    (all t from the old X)

which takes the place of the residual sum X <- X + y.  The model's last norm reads the plain sum of the streams.
``StreamLink`` owns ``in``, ``out`` and ``mix``; the write of one sublayer is handed on as a ``StreamWrite`` and
applied inside the norm that reads the residual next (one pass over the rows: ``ops.stream_tanh_norm``), just as
a pre-norm block folds the residual sum into the next norm.
"""

from __future__ import annotations

from typing import Dict

import torch

from .base import Block, Connection, StreamWrite, TensorDecl, register_part


class StreamLink(Connection):
    def __init__(self, spec):
        super().__init__(spec)
        self.streams = int(spec.params["streams"])
        self.read = self.out = self.mix = None

    def tensors(self) -> Dict[str, TensorDecl]:
        s = self.streams
        return {"in": TensorDecl((s,), "bias", std=0.15, mean=1.0 / s),
                "out": TensorDecl((s,), "bias", std=0.15, mean=1.0),
                "mix": TensorDecl((s, s), "bias", std=0.1, eye=1.0)}

    def load(self, fetch, dtype, device) -> None:
        self.read = fetch("in").to(torch.float32).to(device).contiguous()
        self.out = fetch("out").to(torch.float32).to(device).contiguous()
        self.mix = fetch("mix").to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return 4 * (2 * self.streams + self.streams * self.streams)

    def kernel_libraries(self):
        return ("core", "streams")

    def write(self, y) -> StreamWrite:
        return StreamWrite(y, self.mix, self.out)


class HyperPreNormBlock(Block):
    """Pre-norm over a residual of several streams: the mixer, then the feed-forward, each joined by a link."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_link": "connection",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_link": "connection"}

    def forward(self, h, delta, step, caches):
        x = self.mixer_norm.add_forward(h, delta, read=self.mixer_link.read)
        a = self.mixer.forward(x, step, caches["mixer"])
        x = self.feed_forward_norm.add_forward(h, self.mixer_link.write(a), read=self.feed_forward_link.read)
        f = self.feed_forward.forward(x, step)
        return h, self.feed_forward_link.write(f)


class HyperMixerOnlyBlock(Block):
    """The same for a layer without a feed-forward."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_link": "connection"}

    def forward(self, h, delta, step, caches):
        x = self.mixer_norm.add_forward(h, delta, read=self.mixer_link.read)
        a = self.mixer.forward(x, step, caches["mixer"])
        return h, self.mixer_link.write(a)


register_part("connection", "stream_link", StreamLink)
register_part("block", "hyper_pre_norm", HyperPreNormBlock)
register_part("block", "hyper_mixer_only", HyperMixerOnlyBlock)
