"""GPU tests of the device-side automaton builders (bit-exact against the Python generators of the
synthetic workloads and against torch's own CTC loss) and of the plan cache."""
import numpy as np
import pytest
import torch

from i6_native_ops_b200 import workloads as wl

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods(cuda):
    import i6_native_ops_b200.fbw as fbw
    import i6_native_ops_b200.topology as topo

    return fbw, topo


def python_batch(builders):
    """Concatenate per-sequence (n, fr, to, em, w, start, end) automata with global state ids."""
    fr, to, em, sq, w, st, en = [], [], [], [], [], [], []
    off = 0
    for b, (n, f_, t_, e_, w_, s_, x_) in enumerate(builders):
        fr += [off + v for v in f_]
        to += [off + v for v in t_]
        em += list(e_)
        sq += [b] * len(f_)
        w += list(w_)
        st.append(off + s_)
        en.append(off + x_)
        off += n
    return off, np.array([fr, to, em, sq], dtype=np.int32), np.array(w, dtype=np.float32), \
        np.array([st, en], dtype=np.int32)


def test_ctc_topology_matches_python_builder(mods, cuda):
    _, topo = mods
    rng = np.random.default_rng(5)
    lens = [0, 1, 2, 7, 300, 40, 513]
    Lmax = max(lens)
    labels = np.zeros((len(lens), Lmax), dtype=np.int32)
    for b, L in enumerate(lens):
        labels[b, :L] = rng.integers(1, 6, size=L)  # few symbols: many repeated neighbours (no skip)
    S, edges, weights, start_end = topo.ctc_topology(torch.from_numpy(labels).to(cuda),
                                                     torch.tensor(lens, dtype=torch.int32, device=cuda), blank=0)
    want = python_batch([wl._ctc_fsa(labels[b, :L]) for b, L in enumerate(lens)])
    assert S == want[0]
    assert np.array_equal(edges.cpu().numpy(), want[1])
    assert np.array_equal(weights.cpu().numpy(), want[2])
    assert np.array_equal(start_end.cpu().numpy(), want[3])


@pytest.mark.parametrize("skip,optional", [(None, False), (0.05, False), (None, True)])
def test_hmm_topology_matches_python_builder(mods, cuda, skip, optional):
    _, topo = mods
    rng = np.random.default_rng(9)
    lens = [1, 2, 3, 50, 700, 257]
    Nmax = max(lens)
    classes = rng.integers(0, 1000, size=(len(lens), Nmax)).astype(np.int32)
    opt = (rng.random((len(lens), Nmax)) < 0.3).astype(np.uint8)
    S, edges, weights, start_end = topo.hmm_topology(
        torch.from_numpy(classes).to(cuda), torch.tensor(lens, dtype=torch.int32, device=cuda), 0.3, 0.7,
        skip_prob=skip, optional=torch.from_numpy(opt).to(cuda) if optional else None)
    want = python_batch([wl._chain_hmm(classes[b, :N], opt[b, :N] if optional else [False] * N, 0.3, 0.7, skip)
                         for b, N in enumerate(lens)])
    assert S == want[0]
    assert np.array_equal(edges.cpu().numpy(), want[1])
    assert np.array_equal(weights.cpu().numpy(), want[2])
    assert np.array_equal(start_end.cpu().numpy(), want[3])


def test_ctc_topology_with_fbw_equals_torch_ctc_loss(mods, cuda):
    fbw, topo = mods
    torch.manual_seed(3)
    B, T, F, Lmax = 6, 40, 23, 9
    log_probs = torch.randn(B, T, F, device=cuda).log_softmax(-1)
    label_lens = torch.tensor([3, 9, 1, 5, 7, 2], dtype=torch.int32, device=cuda)
    labels = torch.randint(1, F, (B, Lmax), dtype=torch.int32, device=cuda)
    seq_lens = torch.tensor([40, 33, 25, 40, 38, 12], dtype=torch.int32, device=cuda)
    fsa = topo.ctc_topology(labels, label_lens, blank=0)
    loss = fbw.fbw_loss(log_probs, fsa, seq_lens)  # (T, B); frame 0 holds each sequence's NLL
    want = torch.nn.functional.ctc_loss(log_probs.transpose(0, 1).double().cpu(), labels.long().cpu(),
                                        seq_lens.long().cpu(), label_lens.long().cpu(), blank=0, reduction="none")
    assert torch.allclose(loss[0].double().cpu(), want, rtol=1e-5, atol=1e-5)


def test_plan_cache_reuses_and_invalidates(mods, cuda):
    fbw, _ = mods
    b = wl.make_batch("bpe_ctc", B=8, T=120, F=1025, scale=0.3)
    fsa, sl = wl.to_torch(b, cuda)
    log_probs = (-wl.make_scores(b, cuda)).transpose(0, 1).contiguous()
    cache = fbw.PlanCache(capacity=2)
    x1 = log_probs.clone().requires_grad_(True)
    x2 = log_probs.clone().requires_grad_(True)
    l1 = fbw.fbw_loss(x1, fsa, sl)
    l1.sum().backward()
    l2 = fbw.fbw_loss_cached(x2, fsa, sl, cache)
    l2.sum().backward()
    assert torch.equal(l1, l2) and torch.equal(x1.grad, x2.grad)
    assert (cache.hits, cache.misses) == (0, 1)
    fbw.fbw_loss_cached(x2.detach(), fsa, sl, cache)
    assert (cache.hits, cache.misses) == (1, 1)
    # an in-place change of a key tensor is a different automaton: no stale plan
    w2 = fsa[2]
    w2.add_(0.5)
    l3 = fbw.fbw_loss_cached(x2.detach(), fsa, sl, cache)
    assert (cache.hits, cache.misses) == (1, 2)
    assert torch.equal(l3, fbw.fbw_loss(x2.detach(), fsa, sl))
    assert not torch.equal(l3, l2)
    # capacity: least recently used entries are dropped
    for k in range(3):
        other = wl.make_batch("bpe_ctc", B=8, T=120, F=1025, scale=0.3, seed0=100 + k)
        fo, so = wl.to_torch(other, cuda)
        fbw.fbw_loss_cached(x2.detach(), fo, so, cache)
    assert len(cache._entries) == 2
