"""PackBitsTensor: a batch of boolean feature vectors packed along the batch dimension.

Drop-in for the reference class (difflogic/packbitstensor.py:6-41): `.t` is the packed tensor
`[features, ceil(batch / bit_count)]` of dtype int{bit_count}, `.pad_len` the number of unused
high bits in the last word, sample s being bit s % bit_count (LSB first) of word s // bit_count.

Evaluation is lazy.  A LogicLayer in eval mode does not compute at once; it appends itself to the
tensor's list of pending layers.  Reading `.t` runs the pending layers one kernel per layer, exactly
as the reference does.  `group_sum(k)` -- what GroupSum calls -- runs all pending layers but the last
one kernel each and hands the last layer together with the bit-sum to ONE kernel that never stores the
layer's output (ops.eval_groupbitsum) when the sizes are in that kernel's range.  The counts are
identical either way; the in-place semantics of the reference (the layer returns the same object, `.t`
then holds the layer's output) are kept.
"""
import os

import numpy as np
import torch

from . import ops


# Module switch, read from the environment once at import (set the attribute to change it afterwards).
FUSED_LAST_LAYER = os.environ.get("DL_FUSED_LAST_LAYER", "1") != "0"   # last layer + bit-sum in one kernel


class PackBitsTensor:
    def __init__(self, t: torch.BoolTensor, bit_count=32, device='cuda'):
        assert len(t.shape) == 2, t.shape

        self.bit_count = bit_count
        self.device = device
        self._pending = []

        if device == 'cuda' or (isinstance(device, (str, torch.device)) and torch.device(device).type == 'cuda'):
            t = t.to(device)
            if t.dtype != torch.bool:
                t = t != 0
            # transpose and pack in one kernel, straight from the batch-major matrix
            self._t, self.pad_len = ops.packbits_batch_major(t.contiguous(), self.bit_count)
        else:
            raise NotImplementedError(device)

    @classmethod
    def from_packed(cls, words, pad_len, device='cuda'):
        """Wraps words that are already packed (e.g. a batch shard that was packed elsewhere)."""
        self = cls.__new__(cls)
        self.bit_count = ops.bits_of(words)
        self.device = device
        self._t = words
        self._pending = []
        self.pad_len = int(pad_len)
        return self

    @classmethod
    def from_uint8_thresholds(cls, t, thresholds=(63, 127, 191), bit_count=64, device='cuda'):
        """Thermometer-encodes uint8 features (e.g. images `[batch, C, H, W]`) and packs them in one kernel.
        Feature `i * n + f` of the result is `t[:, f] > thresholds[i]` with f running over the flattened trailing
        dimensions -- the layout of `torch.cat([x > (i+1)/4 ...], dim=1)` followed by Flatten on `x = t / 255`."""
        t = t.to(device).reshape(t.shape[0], -1).contiguous()
        words, pad_len = ops.threshold_packbits_batch_major(t, thresholds, bit_count)
        return cls.from_packed(words, pad_len, device=device)

    # -- lazy layer application ------------------------------------------------------------------

    @property
    def t(self):
        """The packed tensor after every layer applied so far (pending layers run now, one kernel each)."""
        self._materialize()
        return self._t

    @t.setter
    def t(self, value):
        self._pending = []
        self._t = value

    def _push_layer(self, layer):
        """Called by LogicLayer.forward_cuda_eval: remember the layer (its connections and current arg-max gates)."""
        rows = self._pending[-1][0].out_dim if self._pending else self._t.shape[0]
        assert rows == layer.in_dim, ((rows,), layer.in_dim)
        self._pending.append((layer, layer._gate_ids()))

    def _materialize(self):
        pending, self._pending = self._pending, []
        for layer, gate in pending:
            a, b = layer.indices
            self._t = ops.eval_packed(self._t, a, b, gate)

    def group_sum(self, k):
        assert torch.device(self.device).type == 'cuda', self.device
        if self._pending and FUSED_LAST_LAYER:
            # all layers but the last run now; the last one is counted as it is computed, its output never stored
            (layer, gate) = self._pending.pop()
            self._materialize()
            self._pending.append((layer, gate))  # still pending: `.t` would run it as a kernel of its own
            if ops.eval_groupbitsum_applicable(self._t, layer.out_dim, k):
                a, b = layer.indices
                return ops.eval_groupbitsum(self._t, a, b, gate, self.pad_len, k)
        return ops.groupbitsum(self.t, self.pad_len, k)

    def flatten(self, start_dim=0, end_dim=-1, **kwargs):
        """Returns the object itself so that torch.nn.Flatten passes it through; arguments are ignored."""
        return self

    def _row_repr(self, row):
        def word(v):
            return np.binary_repr(int(v), width=self.bit_count)[::-1]
        row = row.tolist()
        if len(row) <= 4:
            return ' '.join(word(v) for v in row)
        return '{} ... {}'.format(' '.join(word(v) for v in row[:3]), word(row[-1]))

    def __repr__(self):
        return '\n'.join(self._row_repr(row) for row in self.t.cpu())
