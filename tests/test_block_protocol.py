"""The block arrangement's hand-over of a norm's work to the product before it
(``parts/block.py``), with stand-in parts that record what they are given: no kernels run."""

import pytest
import torch

from distengine_b200.parts.base import FeedForward, Mixer, Norm
from distengine_b200.parts.block import PreNormBlock
from distengine_b200.parts.context import NormAhead, ResidualStream, UnscaledRows


class _Norm(Norm):
    def __init__(self, name, can_hand_over=True):
        super().__init__(torch.float32, torch.device("cpu"))
        self.name, self.can_hand_over, self.runs = name, can_hand_over, 0

    def forward(self, stream, ctx, rows=None):
        assert stream.ahead is None
        self.runs += 1
        if stream.pending is not None:
            stream.resid += stream.pending
            stream.pending = None
        return stream.resid.clone()

    def ahead(self, stream, ctx, count):
        if not self.can_hand_over or stream.pending is not None:
            return None
        n, width = stream.resid.shape
        return NormAhead(self, stream.resid, torch.ones(width), 1e-5, torch.zeros(n, width),
                         torch.zeros(n, count))


class _Part:
    """A mixer or feed-forward that adds 1 to the stream, through either interface."""

    def __init__(self, name, takes, parts, log):
        self.name, self._takes, self._parts, self.log = name, takes, parts, log

    def takes_unscaled(self, n_rows):
        return self._takes

    def ahead_parts(self, n_rows):
        return self._parts

    def _run(self, x, ahead):
        self.log.append((self.name, type(x).__name__, ahead is not None))
        if ahead is None:
            rows = x.rows if isinstance(x, UnscaledRows) else x
            return torch.ones_like(rows)
        ahead.resid += 1.0
        ahead.rows.copy_(ahead.resid)
        ahead.parts.fill_(1.0)
        return None


class _Mixer(_Part, Mixer):
    def forward(self, x, ctx, cache, ahead=None):
        return self._run(x, ahead)


class _FeedForward(_Part, FeedForward):
    def forward(self, x, ctx, ahead=None):
        return self._run(x, ahead)


class _PlainMixer(Mixer):
    """Says nothing about the optional abilities: the defaults must keep it on plain tensors."""

    def __init__(self, log):
        super().__init__(torch.float32, torch.device("cpu"))
        self.log = log

    def forward(self, x, ctx, cache):
        self.log.append(("plain", type(x).__name__, False))
        return torch.ones_like(x)


def _block(log, mixer_takes, mixer_parts, ffn_takes, ffn_parts, norms=(True, True)):
    n1, n2 = _Norm("n1", norms[0]), _Norm("n2", norms[1])
    block = PreNormBlock(_Mixer("mixer", mixer_takes, mixer_parts, log),
                         _FeedForward("ffn", ffn_takes, ffn_parts, log), n1, n2)
    return block, n1, n2


def test_every_part_able_the_norms_in_between_do_not_run():
    log = []
    first, a1, a2 = _block(log, True, 4, True, 4)
    second, b1, b2 = _block(log, True, 4, True, 4)
    stream = ResidualStream(torch.zeros(3, 8))
    first.forward(stream, None, None, following=(second.mixer_norm, second.mixer))
    second.forward(stream, None, None, following=None)
    # only the very first norm runs; the last feed-forward has nobody to hand over to
    assert (a1.runs, a2.runs, b1.runs, b2.runs) == (1, 0, 0, 0)
    assert log == [("mixer", "Tensor", True), ("ffn", "UnscaledRows", True),
                   ("mixer", "UnscaledRows", True), ("ffn", "UnscaledRows", False)]
    assert stream.ahead is None and stream.pending is not None
    assert torch.equal(stream.resid + stream.pending, torch.full((3, 8), 4.0))


def test_a_part_without_the_abilities_gets_plain_tensors():
    log = []
    n1, n2 = _Norm("n1"), _Norm("n2")
    block = PreNormBlock(_PlainMixer(log), _FeedForward("ffn", True, 4, log), n1, n2)
    stream = ResidualStream(torch.zeros(2, 8))
    block.forward(stream, None, None, following=(n1, block.mixer))     # a mixer that cannot take it
    assert (n1.runs, n2.runs) == (1, 1)
    assert log == [("plain", "Tensor", False), ("ffn", "Tensor", False)]
    assert stream.ahead is None


@pytest.mark.parametrize("mixer_parts,ffn_takes,norm_can", [(0, True, True), (4, False, True),
                                                            (4, True, False)])
def test_producer_consumer_and_norm_must_all_be_able(mixer_parts, ffn_takes, norm_can):
    log = []
    block, n1, n2 = _block(log, True, mixer_parts, ffn_takes, 0, norms=(True, norm_can))
    stream = ResidualStream(torch.zeros(2, 8))
    block.forward(stream, None, None)
    assert n2.runs == 1 and log[0] == ("mixer", "Tensor", False) and log[1][1] == "Tensor"


def test_another_norms_work_is_not_taken_for_ones_own():
    log = []
    block, n1, n2 = _block(log, True, 4, True, 4)
    stream = ResidualStream(torch.zeros(2, 8))
    stranger = _Norm("other")
    stream.ahead = stranger.ahead(stream, None, 4)
    with pytest.raises(RuntimeError, match="another norm"):
        block.forward(stream, None, None)
