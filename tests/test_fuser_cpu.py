"""The fuser's host logic without a GPU: region limits, the walk over shared subexpressions, and the graph
matchers that turn a softmax / LayerNorm written from primitives into one row kernel. Leaves are stand-in nodes;
what would be evaluated on the device is replaced by CPU buffers of the right shape."""
import pytest
import torch

from pequegrad_b200 import _lib as L
from pequegrad_b200 import fuser
from pequegrad_b200 import tensor as pg


def leaf(shape=(4, 5), dtype=torch.float32):
    return pg.Tensor(op="input", shape=shape, dtype=dtype)


@pytest.fixture
def fake_device(monkeypatch):
    """`_emit_leaf` without a device: inputs get a CPU buffer; an elementwise node that the region limits cut off is
    built as a region of its own, which must fit, and then counts as evaluated."""
    regions = []

    def emit_leaf(node, fuse):
        if node._buf is None:
            if node.op in fuser._ELEMENTWISE and node.op != "fill":
                reg = fuser._Region(node.shape, fuse)
                reg.emit(node)
                assert reg.fits() and len(reg.prog) <= L.MAX_INSTRS and len(reg.inputs) <= L.MAX_INPUTS
                regions.append(reg)
            node._buf = torch.empty(node.shape, dtype=node.dtype)
        return node._buf

    monkeypatch.setattr(fuser, "_emit_leaf", emit_leaf)
    return regions


def build(node, fake):
    reg = fuser._Region(node.shape, fuser.JIT)
    reg.emit(node)
    assert reg.fits() and len(reg.prog) <= L.MAX_INSTRS and len(reg.inputs) <= L.MAX_INPUTS
    return reg


def test_a_sum_of_ten_tensors_is_split_at_the_input_limit(fake_device):
    xs = [leaf() for _ in range(10)]
    acc = xs[0]
    for x in xs[1:]:
        acc = acc + x  # left-deep: every node is entered before any operand is emitted
    reg = build(acc, fake_device)
    assert len(reg.inputs) <= L.MAX_INPUTS and len(fake_device) >= 1  # at least one subtree became a region of its own


def test_a_chain_of_forty_ops_is_split_at_the_instruction_limit(fake_device):
    x = leaf()
    y = x
    for _ in range(40):
        y = (y * 1.5).exp() if _ % 2 else y + 1.0
    reg = build(y, fake_device)
    assert len(reg.prog) <= fuser.MAX_REGION_INSTRS
    total = len(reg.prog) + sum(len(r.prog) for r in fake_device)
    assert total >= 40  # nothing was dropped


def test_balanced_tree_and_where_fit_after_cutting(fake_device):
    xs = [leaf() for _ in range(16)]
    level = xs
    while len(level) > 1:
        level = [pg.where(a > b, a, b) * 2.0 for a, b in zip(level[::2], level[1::2])]
    build(level[0], fake_device)


def test_shared_subexpressions_are_walked_once():
    # y = y + y thirty times: 2^30 paths through the DAG, 31 nodes
    y = leaf()
    for _ in range(30):
        y = y + y
    assert fuser._find_reduce(y, y.shape) is None  # returns at once instead of walking every path
    r = (leaf((4, 5)).sum(1, True))
    z = pg.broadcast_to(r, (4, 1))
    for _ in range(30):
        z = z * z
    assert fuser._find_reduce(z, z.shape) is r
    assert fuser._subtree_size(y, y.shape) == 31


def test_softmax_and_layernorm_written_from_primitives_are_recognised():
    x = leaf((8, 1024))
    assert fuser._match_softmax(pg.softmax(x)) is x
    m = x.max_reduce(-1, True)
    e = (x - m).exp()
    assert fuser._match_softmax(e / e.sum(-1, True)) is x          # written by hand
    assert fuser._match_softmax(e / e.sum(0, True)) is None         # another axis: not the row kernel's case
    assert fuser._match_softmax(e / (e.sum(-1, True) + 1.0)) is None
    assert fuser._match_softmax((x - 1.0).exp() / e.sum(-1, True)) is None
    w, b = leaf((1024,)), leaf((1024,))
    for weight, bias in ((None, None), (w, None), (w, b)):
        got = fuser._match_layernorm(pg.layer_norm(x, 1024, 1e-5, weight, bias))
        assert got is not None and got[0] is x and got[1] is weight and got[2] is bias and got[3] == 1e-5 and got[4] == 1024
    x3 = leaf((2, 3, 4))
    got = fuser._match_layernorm(pg.layer_norm(x3, (3, 4)))
    assert got is not None and got[4] == 12
    # by hand, with the variance written out
    mu = x.mean(-1, True)
    var = ((x - mu) ** 2.0).sum(-1, True) / 1024.0
    assert fuser._match_layernorm((x - mu) / (var + 1e-6) ** 0.5 * w)[3] == 1e-6
    assert fuser._match_layernorm((x - mu) / (var + 1e-6) ** 0.5 * 2.0) is None   # a scalar is not a weight vector
    var_unbiased = ((x - mu) ** 2.0).sum(-1, True) / 1023.0
    assert fuser._match_layernorm((x - mu) / (var_unbiased + 1e-6) ** 0.5) is None  # not LayerNorm's variance
    assert fuser._match_layernorm(x * w + b) is None
