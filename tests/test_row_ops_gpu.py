"""Row-wise sm_100a kernels against their eager PyTorch oracles (forward and backward)."""
import pytest
import torch

from lset_b200.ops import _native as nv
from lset_b200.ops import activation as A
from lset_b200.ops import embedding as E
from lset_b200.ops import norm as N
from lset_b200.ops import pooling as P
from lset_b200.ops import rope as R

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(BF)


def _close(a, b, tol=2e-2, name=""):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item() + 1e-6
    assert err / ref < tol, f"{name}: err {err:.4g} ref {ref:.4g}"


def _grads(fn, inputs, gout):
    leaves = [t.detach().clone().requires_grad_() for t in inputs]
    out = fn(*leaves)
    outs = out if isinstance(out, tuple) else (out,)
    gs = gout if isinstance(gout, tuple) else (gout,)
    torch.autograd.backward([o for o in outs if o is not None], [g for g in gs])
    return outs, [l.grad for l in leaves]


def _f32(fn):
    """Run an oracle in fp32 on fp32 copies of bf16 inputs (less rounding noise in the reference)."""
    return fn


@pytest.mark.parametrize("N_,H", [(300, 1024), (1000, 2560), (77, 4096), (513, 768), (64, 128), (9, 8192)])
@pytest.mark.parametrize("w_off", [0.0, 1.0])
def test_rms_norm(N_, H, w_off):
    x, w, g = _r(N_, H), _r(H, scale=0.5), _r(N_, H)
    (y,), gr = _grads(lambda a, b: N.rms_norm(a, b, 1e-6, w_off), [x, w], g)
    (yr,), grr = _grads(lambda a, b: N.rms_norm_ref(a, b, 1e-6, w_off), [x.float(), w.float()], g.float())
    nv.check_status()
    _close(y, yr, name="y")
    _close(gr[0], grr[0], name="dx")
    _close(gr[1], grr[1], 3e-2, name="dw")


@pytest.mark.parametrize("N_,H", [(300, 1024), (1000, 2560), (130, 4096)])
def test_residual_rms_norm(N_, H):
    r, x, w = _r(N_, H), _r(N_, H), _r(H, scale=0.5)
    g1, g2 = _r(N_, H), _r(N_, H)
    (y, nr), gr = _grads(lambda a, b, c: N.residual_rms_norm(a, b, c, 1e-6), [r, x, w], (g1, g2))
    (yr, nrr), grr = _grads(lambda a, b, c: N.residual_rms_norm_ref(a, b, c, 1e-6),
                            [r.float(), x.float(), w.float()], (g1.float(), g2.float()))
    _close(y, yr, name="y"); _close(nr, nrr, name="nr")
    _close(gr[0], grr[0], name="dr"); _close(gr[1], grr[1], name="dx"); _close(gr[2], grr[2], 3e-2, name="dw")


@pytest.mark.parametrize("N_,H", [(200, 768), (1000, 1024), (33, 2560)])
def test_double_residual_rms_norm(N_, H):
    r, a, w1, w2 = _r(N_, H), _r(N_, H), _r(H, scale=0.3), _r(H, scale=0.3)
    g1, g2 = _r(N_, H), _r(N_, H)
    (out, nr), gr = _grads(lambda p, q, u, v: N.double_residual_rms_norm(p, q, u, v, 1e-6, 1.0),
                           [r, a, w1, w2], (g1, g2))
    (outr, nrr), grr = _grads(lambda p, q, u, v: N.double_residual_rms_norm_ref(p, q, u, v, 1e-6, 1.0),
                              [t.float() for t in (r, a, w1, w2)], (g1.float(), g2.float()))
    _close(out, outr, name="y"); _close(nr, nrr, name="nr")
    _close(gr[0], grr[0], name="dr"); _close(gr[1], grr[1], 3e-2, name="da")
    _close(gr[2], grr[2], 4e-2, name="dw1"); _close(gr[3], grr[3], 4e-2, name="dw2")


@pytest.mark.parametrize("N_,H", [(300, 768), (1000, 1024), (64, 384)])
@pytest.mark.parametrize("res", [False, True])
def test_layer_norm(N_, H, res):
    x, w, b, g = _r(N_, H), _r(H, scale=0.5), _r(H, scale=0.5), _r(N_, H)
    if res:
        r, g2 = _r(N_, H), _r(N_, H)
        (y, nr), gr = _grads(lambda a, c, d, e: N.residual_layer_norm(a, c, d, e, 1e-12), [r, x, w, b], (g, g2))
        (yr, nrr), grr = _grads(lambda a, c, d, e: N.residual_layer_norm_ref(a, c, d, e, 1e-12),
                                [t.float() for t in (r, x, w, b)], (g.float(), g2.float()))
        _close(nr, nrr, name="nr")
    else:
        (y,), gr = _grads(lambda c, d, e: N.layer_norm(c, d, e, 1e-12), [x, w, b], g)
        (yr,), grr = _grads(lambda c, d, e: N.layer_norm_ref(c, d, e, 1e-12),
                            [t.float() for t in (x, w, b)], g.float())
    _close(y, yr, name="y")
    for i, (a_, b_) in enumerate(zip(gr, grr)):
        _close(a_, b_, 3e-2, name=f"grad{i}")


@pytest.mark.parametrize("Hq,Hk,hd", [(16, 8, 128), (32, 8, 128), (12, 12, 64), (4, 1, 256)])
@pytest.mark.parametrize("do_norm", [True, False])
def test_qk_norm_rope(Hq, Hk, hd, do_norm):
    T = 333
    qkv = _r(T, Hq + 2 * Hk, hd)
    q, k = qkv[:, :Hq], qkv[:, Hq:Hq + Hk]
    qw = _r(hd, scale=0.5) if do_norm else None
    kw = _r(hd, scale=0.5) if do_norm else None
    pos = torch.randint(0, 700, (T,), device="cuda")
    cos, sin = R.rope_tables(hd, 1024, 1e6, "cuda")
    gq, gk = _r(T, Hq, hd), _r(T, Hk, hd)
    ins = [q, k] + ([qw, kw] if do_norm else [])
    f = (lambda a, b, c, d: R.qk_norm_rope(a, b, c, d, cos, sin, pos)) if do_norm else \
        (lambda a, b: R.qk_norm_rope(a, b, None, None, cos, sin, pos))
    fr = (lambda a, b, c, d: R.qk_norm_rope_ref(a, b, c, d, cos, sin, pos)) if do_norm else \
        (lambda a, b: R.qk_norm_rope_ref(a, b, None, None, cos, sin, pos))
    (qo, ko), gr = _grads(f, ins, (gq, gk))
    (qr, kr), grr = _grads(fr, [t.float() for t in ins], (gq.float(), gk.float()))
    nv.check_status()
    _close(qo, qr, name="q"); _close(ko, kr, name="k")
    for i, (a_, b_) in enumerate(zip(gr, grr)):
        _close(a_, b_, 3e-2, name=f"grad{i}")


@pytest.mark.parametrize("kind", ["swiglu", "geglu"])
def test_glu(kind):
    gu, g = _r(500, 2 * 3072), _r(500, 3072)
    (y,), gr = _grads(lambda a: A.glu(a, kind), [gu], g)
    (yr,), grr = _grads(lambda a: A.glu_ref(a[:, :3072], a[:, 3072:], kind), [gu.float()], g.float())
    _close(y, yr); _close(gr[0], grr[0])


def test_gelu():
    x, g = _r(100, 3072), _r(100, 3072)
    (y,), gr = _grads(A.gelu, [x], g)
    (yr,), grr = _grads(torch.nn.functional.gelu, [x.float()], g.float())
    _close(y, yr); _close(gr[0], grr[0])


def test_normalize_and_gather():
    x, g = _r(1500, 1024), _r(1500, 1024)
    (y,), gr = _grads(P.normalize, [x], g)
    (yr,), grr = _grads(lambda a: torch.nn.functional.normalize(a, dim=-1), [x.float()], g.float())
    _close(y, yr); _close(gr[0], grr[0])
    idx = torch.tensor([5, 17, 1499, 0, 700], device="cuda")
    g2 = _r(5, 1024)
    (y2,), gr2 = _grads(lambda a: P.gather_normalize(a, idx), [x], g2)
    (y2r,), gr2r = _grads(lambda a: torch.nn.functional.normalize(a[idx], dim=-1), [x.float()], g2.float())
    _close(y2, y2r); _close(gr2[0], gr2r[0])


@pytest.mark.parametrize("strategy", ["last_token", "cls", "mean", "weighted_mean"])
def test_packed_pool(strategy):
    lens = [5, 130, 64, 1, 300]
    T = sum(lens)
    cu = torch.tensor([0, 5, 135, 199, 200, 500], dtype=torch.int32, device="cuda")
    h, g = _r(T, 768), _r(5, 768)
    (y,), gr = _grads(lambda a: P.packed_pool(a, cu, strategy), [h], g)
    (yr,), grr = _grads(lambda a: P.packed_pool(a, cu, strategy), [h.float()], g.float())
    _close(y, yr); _close(gr[0], grr[0])


def test_embedding():
    tab = _r(1000, 1024).requires_grad_()
    ids = torch.randint(0, 1000, (7, 33), device="cuda")
    out = E.embedding(ids, tab)
    assert torch.equal(out, tab.detach()[ids])
    g = _r(7, 33, 1024)
    out.backward(g)
    ref = torch.zeros(1000, 1024, device="cuda").index_add_(0, ids.reshape(-1), g.reshape(-1, 1024).float())
    _close(tab.grad, ref)
    pos_tab, typ_tab = _r(64, 1024), _r(2, 1024)
    pos = torch.arange(33, device="cuda")[None]
    typ = torch.zeros(7, 33, dtype=torch.long, device="cuda")
    out3 = E.embedding(ids, tab.detach(), extra=((pos, pos_tab), (typ, typ_tab)))
    ref3 = tab.detach()[ids].float() + pos_tab[pos].float() + typ_tab[typ].float()
    _close(out3, ref3)


def test_bounded_wait_times_out_with_status_and_context_survives():
    import ctypes

    lib = nv.load()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")      # nothing ever sets it
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    rc = lib.lb_bounded_wait_probe(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(1),
                                   ctypes.c_ulonglong(200_000_000), ctypes.c_void_p(status.data_ptr()),
                                   ctypes.c_void_p(waited.data_ptr()),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert status.item() == 4 and 0.15e9 < waited.item() < 2e9
    flag.fill_(1)                                                 # a set flag returns at once
    status.zero_()
    lib.lb_bounded_wait_probe(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(1),
                              ctypes.c_ulonglong(200_000_000), ctypes.c_void_p(status.data_ptr()),
                              ctypes.c_void_p(waited.data_ptr()),
                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert status.item() == 0 and waited.item() < 50_000_000
    assert torch.ones(4, device="cuda").sum().item() == 4.0       # the context is still usable


def test_device_barrier_single_gpu_forms():
    """The device barrier on one GPU: a one-rank group passes at once; a two-rank group whose peer
    never announces runs into the bounded wait and reports the peer-timeout status (nothing hangs,
    the context stays usable). The peer's pad is a second local buffer, so no other GPU is involved."""
    import ctypes

    lib = nv.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    peer = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pads1 = (ctypes.c_void_p * 1)(mine.data_ptr())
    for epoch in (1, 2, 3):
        rc = lib.lb_device_barrier(pads1, ctypes.c_int(1), ctypes.c_int(0), ctypes.c_uint(epoch),
                                   ctypes.c_ulonglong(200_000_000),
                                   ctypes.c_void_p(status.data_ptr()), stream)
        assert rc == 0
    torch.cuda.synchronize()
    assert status.item() == 0 and mine[0].item() == 3
    pads2 = (ctypes.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    mine.zero_()
    rc = lib.lb_device_barrier(pads2, ctypes.c_int(2), ctypes.c_int(0), ctypes.c_uint(1),
                               ctypes.c_ulonglong(200_000_000), ctypes.c_void_p(status.data_ptr()),
                               stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert status.item() == 4                      # kStatusTimeoutPeer
    assert mine[0].item() == 1 and peer[0].item() == 1   # this rank did announce to both pads
    mine[1] = 2                                    # the "peer" is already one barrier ahead
    status.zero_()
    lib.lb_device_barrier(pads2, ctypes.c_int(2), ctypes.c_int(0), ctypes.c_uint(2),
                          ctypes.c_ulonglong(200_000_000), ctypes.c_void_p(status.data_ptr()), stream)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_poll_status_raises_one_call_late_without_blocking():
    """The training loop's non-blocking status check: the value seen is the one copied by the
    previous call; a non-zero status raises and clears the word."""
    word = nv.status_word(torch.device("cuda", torch.cuda.current_device()))
    word.zero_()
    nv.poll_status()
    nv.poll_status()                       # still clean
    word.fill_(4)                          # what a kernel that gave up waiting for a peer writes
    nv.poll_status()                       # copies the 4 ...
    with pytest.raises(nv.NativeError):
        nv.poll_status()                   # ... and the next call sees it
    torch.cuda.synchronize()
    assert word.item() == 0
    nv.poll_status()
    nv.poll_status()
