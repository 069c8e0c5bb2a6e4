"""The reference pins ``flash-attn>=2.5,<2.7``; the image ships 2.8, whose ``flash_attn.layers.rotary.RotaryEmbedding``
no longer takes ``pos_idx_in_fp32`` (the reference passes it positionally, src/nanotron/nn/rotary.py:161-168).
``apply()`` restores the 2.6 constructor signature on the installed class; nothing else is touched."""
import inspect


def apply():
    import flash_attn.layers.rotary as rotary

    cls = rotary.RotaryEmbedding
    if "pos_idx_in_fp32" in inspect.signature(cls.__init__).parameters:
        return
    orig = cls.__init__

    def __init__(self, dim, base=10000.0, interleaved=False, scale_base=None, pos_idx_in_fp32=True, device=None):
        orig(self, dim, base=base, interleaved=interleaved, scale_base=scale_base, device=device)
        self.pos_idx_in_fp32 = pos_idx_in_fp32

    cls.__init__ = __init__
