"""Pre-norm residual block: `h += mixer(norm(h))`, then `h += feed_forward(norm(h))`
(src/minillm/runtime.cpp:245-337; src/minillm/cuda/layer.cpp:42-70).

Each residual add is folded into a neighbouring kernel: either the sub-layer's last
product adds its result into `h` itself (it finds `h` in `step.residual` and returns
None), or its output is handed on as `pending` and added to `h` by the next norm's
kernel.  Either way the residual stream is read and written once per sub-layer.  Norm
slots: "pre_mixer", "pre_feed_forward".
"""
from __future__ import annotations

from ..config.registry import register_part
from .base import Block


class PreNormBlock(Block):
    def forward(self, h, pending, step, run):
        step.residual = h
        x = self.norms["pre_mixer"].forward(h, pending, step)
        mixed = self.mixer.forward(x, step, run)
        x = self.norms["pre_feed_forward"].forward(h, mixed, step)
        return self.feed_forward.forward(x, step)

    def first_norm(self):
        return self.norms["pre_mixer"]

    def emit(self, b, h, pending, run):
        b.residual = h
        after = b.norm_after_block
        x = self.norms["pre_mixer"].emit(b, h, pending)
        # Whoever adds into the stream is told which norm reads it next (a few-row product can leave it half done).
        b.norm_ahead = self.norms["pre_feed_forward"].foldable()
        mixed = self.mixer.emit(b, x, run)
        x = self.norms["pre_feed_forward"].emit(b, h, mixed)
        b.norm_ahead = after
        out = self.feed_forward.emit(b, x)
        b.norm_ahead = None
        return out


register_part("block", "pre_norm", PreNormBlock)
