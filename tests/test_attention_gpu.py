"""The fused attention kernel (scores, softmax and PV in one launch) against the fp32 composite of the
reference's GPT-2 block (examples/gpt2.py:168-186), through the C ABI. Tolerance 2e-2 (16-bit inputs)."""
import math

import numpy as np
import pytest
import torch

from pequegrad_b200 import kernels as K

pytestmark = pytest.mark.gpu


def composite(q, k, v, causal, scale):
    s = (q.float() @ k.float().transpose(-2, -1)) * scale
    if causal:
        T, Tk = s.shape[-2:]
        s = s.masked_fill(~torch.tril(torch.ones(T, Tk, dtype=torch.bool, device=s.device)), float("-inf"))
    return torch.softmax(s, -1) @ v.float()


def check(got, want, what):
    err = (got.float() - want).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.abs().max().item()), f"{what}: max abs error {err}"
    assert K.device_error() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,T,causal", [(1, 1, 128, False), (2, 3, 256, True), (1, 2, 1024, True), (2, 2, 200, True),
                                          (1, 2, 72, False), (3, 1, 1, True), (1, 1, 65, True), (1, 4, 129, False)])
def test_attention_matches_the_composite(B, H, T, causal, dtype):
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn((B, H, T, 64), generator=g, device="cuda").to(dtype) for _ in range(3))
    check(K.attention(q, k, v, causal=causal), composite(q, k, v, causal, 0.125), f"{B}x{H}x{T}")


def test_large_scores_and_scale():
    # scores of magnitude ~50: the running max moves between key blocks, so the rows of O are rescaled in tensor memory
    g = torch.Generator(device="cuda").manual_seed(4)
    q, k, v = (torch.randn((2, 2, 512, 64), generator=g, device="cuda") for _ in range(3))
    q, k, v = (q * 3).half(), (k * 3).half(), v.half()
    for scale in (0.125, 0.5):
        check(K.attention(q, k, v, scale=scale, causal=True), composite(q, k, v, True, scale), f"scale {scale}")
    # keys sorted so that every later block raises the max of every row
    k2 = (torch.arange(512, device="cuda").float()[None, None, :, None] * 0.02 * torch.ones(64, device="cuda")).half().expand(2, 2, 512, 64).contiguous()
    q2 = torch.ones((2, 2, 512, 64), device="cuda").half()
    check(K.attention(q2, k2, v, causal=False), composite(q2, k2, v, False, 0.125), "monotone keys")


def test_heads_inside_packed_buffers_and_cross_lengths():
    # q, k, v as slices of a packed [B, T, 3C] buffer, output written into [B, T, C]: the GPT-2 layout
    B, T, H = 2, 384, 12
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = torch.randn((B, T, 3 * H * 64), generator=g, device="cuda").half()
    q, k, v = (qkv[:, :, i * H * 64:(i + 1) * H * 64].view(B, T, H, 64).permute(0, 2, 1, 3) for i in range(3))
    y = torch.zeros((B, T, H * 64), device="cuda", dtype=torch.float16)
    K.attention(q, k, v, causal=True, out=y.view(B, T, H, 64).permute(0, 2, 1, 3))
    want = composite(q, k, v, True, 0.125).permute(0, 2, 1, 3).reshape(B, T, H * 64)
    check(y, want, "packed")
    # more keys than queries, no mask; 3-D tensors
    q3 = torch.randn((4, 100, 64), generator=g, device="cuda").half()
    k3, v3 = (torch.randn((4, 300, 64), generator=g, device="cuda").half() for _ in range(2))
    check(K.attention(q3, k3, v3), composite(q3, k3, v3, False, 0.125), "cross lengths")


@pytest.mark.parametrize("B,H,T,Tk,causal,dtype", [(4, 12, 1024, 1024, True, torch.float16), (50, 12, 128, 128, True, torch.float16),
                                                   (3, 40, 300, 384, False, torch.bfloat16), (7, 12, 200, 200, True, torch.float16),
                                                   (40, 16, 1, 130, False, torch.float16), (12, 12, 1024, 1024, True, torch.float16),
                                                   (100, 12, 100, 100, True, torch.bfloat16)])
def test_more_work_items_than_resident_ctas(B, H, T, Tk, causal, dtype):
    # The kernel is persistent (two CTAs per SM): with more (batch, head, query block) items than CTAs every CTA walks
    # several items back to back, with its loads and MMAs already in the next item while the softmax of the current one
    # finishes and the previous item's result written out inside the next item's first block. Items of one key block,
    # of several, ragged last blocks and a different mix per CTA; up to three items per CTA are handed out in rounds of
    # alternating direction, more in the plain order (the last two cases).
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn((B, H, T, 64), generator=g, device="cuda").to(dtype)
    k, v = (torch.randn((B, H, Tk, 64), generator=g, device="cuda").to(dtype) for _ in range(2))
    out = torch.full((B, H, T, 64), float("nan"), device="cuda", dtype=dtype)
    K.attention(q, k, v, causal=causal, out=out)
    for lo in range(0, B, 8):  # the composite materialises [b, H, T, Tk] fp32 scores: a few batches at a time
        check(out[lo:lo + 8], composite(q[lo:lo + 8], k[lo:lo + 8], v[lo:lo + 8], causal, 0.125), f"batches {lo}..")
    # the same call again gives the same bits (nothing depends on which CTA took which item)
    out2 = torch.empty_like(out)
    K.attention(q, k, v, causal=causal, out=out2)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """Failure detection without a fault: the next attention launch's producer is told to load nothing and every wait
    to give up after 1024 polls. Every CTA must record who gave up, drain its roles, free its tensor memory and return;
    while the error word is set further launches do nothing; after the reset the same call is right again."""
    import ctypes as C

    from pequegrad_b200 import _lib as L
    g = torch.Generator(device="cuda").manual_seed(17)
    q, k, v = (torch.randn((2, 3, 384, 64), generator=g, device="cuda").half() for _ in range(3))
    want = composite(q, k, v, True, 0.125)
    check(K.attention(q, k, v, causal=True), want, "before the drill")
    K.gemm_wait_drill(1024, skip_loads=True)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.float16)
    K.attention(q, k, v, causal=True, out=out)
    torch.cuda.synchronize()  # returns: nothing hangs
    code = C.c_int(0)
    st = L.lib().pgb_device_error(C.byref(code), 0)
    assert st == L.ERR_TIMEOUT and "wait ran out" in L.lib().pgb_last_error().decode()
    assert 16 <= (code.value >> 16) <= 26 and (code.value & 0xffff) < 2 * 3 * 3  # an attention role of one of the 18 CTAs
    assert (out == 7).all()  # nothing was computed, nothing was written
    # the word is still set: the next launch returns at once and leaves its output alone
    K.attention(q, k, v, causal=True, out=out)
    torch.cuda.synchronize()
    assert (out == 7).all()
    assert K.device_error(reset=True) == code.value
    assert K.device_error() == 0
    # the drill applied to one launch only, and the device is as good as before
    check(K.attention(q, k, v, causal=True), want, "after the drill")
    x = torch.randn((256, 512), generator=g, device="cuda").half()
    y = torch.randn((384, 512), generator=g, device="cuda").half()
    assert torch.allclose(K.matmul(x, y.T).float(), x.float() @ y.float().T, rtol=2e-2, atol=2e-2)


def test_attention_errors():
    q = torch.zeros((1, 1, 16, 32), device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="head dim of 64"):
        K.attention(q, q, q)
    q = torch.zeros((1, 1, 16, 64), device="cuda", dtype=torch.float32)
    with pytest.raises(RuntimeError, match="not implemented for"):
        K.attention(q, q, q)
    q = torch.zeros((1, 1, 16, 64), device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match="disagree"):
        K.attention(q, q[:, :, :8], q)
    with pytest.raises(ValueError, match="scale"):
        K.attention(q, q, q, scale=-1.0)
