"""The CUDA-graph cache on a GPU: one capture per shape, replay equal to the eager
forward, refilled inputs, the policy matrix, prewarm, the failed-capture sentinel and
the refusal to nest captures - the cases the reference pins in
``backend/tests/test_cuda_graph_capture.py:60-190`` - plus the ownership of the
scratch memory a captured graph writes: many entries with growing shapes, then the
earliest ones replayed again."""

import pytest
import torch

from helpers import make_case

pytestmark = pytest.mark.gpu


@pytest.fixture()
def gc():
    from zip_kernel_b200.backend import graph_cache as m
    prev = m.get_cuda_graph_policy()
    m.clear_cuda_graph_cache()
    m._cache = m._GraphCache()
    m.set_cuda_graph_policy("off")
    yield m
    m.clear_cuda_graph_cache()
    m._cache = m._GraphCache()
    m.set_cuda_graph_policy(prev)


@pytest.fixture(scope="module")
def small():
    W, X = make_case(1, 2048, 2048, 0.1, perm_seed=3)
    return X.cuda(), W.to(torch.device("cuda"))


def eager(X, W):
    from zip_kernel_b200 import v9_linear
    return v9_linear.v9_linear_forward(X, W)


def test_capture_replay_equals_eager_and_refilled_input(gc, small):
    X, W = small
    y_eager = eager(X, W)
    gc.set_cuda_graph_policy("force")
    y = gc.v9_linear_forward_cuda_graph(X, W)
    st = gc.cuda_graph_cache_stats()
    assert st["n_entries"] == 1 and st["n_capture_fail"] == 0 and st["n_miss"] == 1
    assert torch.equal(y, y_eager)                     # same kernels, same inputs: same bits
    # second call replays (one more hit, no new entry) and sees the NEW contents of X
    X2 = (X.float() * -0.5 + 0.25).half()
    y2 = gc.v9_linear_forward_cuda_graph(X2, W)
    st2 = gc.cuda_graph_cache_stats()
    assert st2["n_entries"] == 1 and st2["n_hit"] == st["n_hit"] + 1
    assert torch.equal(y2, eager(X2, W))
    assert not torch.equal(y2, y)
    assert torch.equal(y, y_eager), "an earlier result must not alias the graph's output buffer"


def test_distinct_shapes_capture_once_each_and_prewarm(gc, small):
    X1, W = small
    X2 = torch.cat([X1, X1 * 0.5]).contiguous()
    X4 = torch.cat([X2, X2 * 0.25]).contiguous()
    gc.set_cuda_graph_policy("force")
    res = gc.prewarm_cuda_graph_cache([(X1, W), (X2, W), (X4, W)])
    assert res == {"attempted": 3, "captured": 3, "skipped": 0}
    assert gc.cuda_graph_cache_stats()["n_entries"] == 3
    for X in (X1, X2, X4):
        assert torch.equal(gc.v9_linear_forward_cuda_graph(X, W), eager(X, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 3     # all replays
    X3d = X4.reshape(2, 2, -1)                                # leading dims are part of the key
    y3 = gc.v9_linear_forward_cuda_graph(X3d, W)
    assert y3.shape == (2, 2, W.d_out) and torch.equal(y3.reshape(4, -1), eager(X4, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 4


def test_policy_off_and_auto_buckets(gc, small):
    X1, W = small
    assert torch.equal(gc.v9_linear_forward_cuda_graph(X1, W), eager(X1, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 0       # off: nothing captured
    gc.set_cuda_graph_policy("auto")
    X3 = torch.cat([X1, X1, X1]).contiguous()                  # 3 is not a power of two: eager under auto
    X8 = torch.cat([X1] * 8).contiguous()
    X200 = torch.cat([X1] * 200).contiguous()                  # beyond the decode threshold: always eager
    assert torch.equal(gc.v9_linear_forward_cuda_graph(X3, W), eager(X3, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 0
    assert torch.equal(gc.v9_linear_forward_cuda_graph(X8, W), eager(X8, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 1
    gc.set_cuda_graph_policy("force")
    assert torch.equal(gc.v9_linear_forward_cuda_graph(X3, W), eager(X3, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 2
    assert torch.equal(gc.v9_linear_forward_cuda_graph(X200, W), eager(X200, W))
    assert gc.cuda_graph_cache_stats()["n_entries"] == 2


def test_failed_capture_leaves_a_sentinel(gc, small, monkeypatch):
    X, W = small
    gc.set_cuda_graph_policy("force")

    class Poison:
        def __init__(self, *a, **kw):
            pass

        def __enter__(self):
            raise RuntimeError("synthetic capture failure")

        def __exit__(self, *a):
            return False

    monkeypatch.setattr(torch.cuda, "graph", Poison)
    y = gc.v9_linear_forward_cuda_graph(X, W)                 # must not raise: falls back to eager
    st = gc.cuda_graph_cache_stats()
    assert st["n_capture_fail"] == 1 and st["n_entries"] == 1
    gc.v9_linear_forward_cuda_graph(X, W)                      # no second attempt
    assert gc.cuda_graph_cache_stats()["n_capture_fail"] == 1
    monkeypatch.undo()
    assert torch.equal(y, eager(X, W))


def test_nested_capture_is_refused(gc, small, monkeypatch):
    X, W = small
    eager(X, W)                       # sizes the shared scratch before the capture state is faked
    gc.set_cuda_graph_policy("force")
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    gc.v9_linear_forward_cuda_graph(X, W)
    st = gc.cuda_graph_cache_stats()
    assert st["n_capture_fail"] == 1 and st["n_entries"] == 1


def test_many_entries_with_growing_shapes_keep_their_scratch(gc):
    """Each captured graph owns the scratch its kernels write.  More entries than torch has pooled
    stream handles (32), with growing token counts and input widths - so later captures need more
    scratch than earlier ones - and then the EARLIEST entries are replayed and compared with eager."""
    gc._cache = gc._GraphCache(capacity=128)
    gc.set_cuda_graph_policy("force")
    dev = torch.device("cuda")
    cases = []
    for K in (256, 512, 1024, 2048):
        W, _ = make_case(1, 384, K, 0.2, perm_seed=K)
        Wd = W.to(dev)
        for T in (1, 2, 3, 5, 8, 13, 16, 24, 32, 48):
            g = torch.Generator().manual_seed(T * 7 + K)
            X = (torch.randn(T, K, generator=g)).half().to(dev)
            cases.append((X, Wd))
    assert len(cases) == 40
    first = [gc.v9_linear_forward_cuda_graph(X, W) for X, W in cases]
    assert gc.cuda_graph_cache_stats()["n_entries"] == 40
    torch.cuda.synchronize()
    # a large eager call on the shared cache in between (grows and replaces the shared scratch)
    Wb, Xb = make_case(128, 512, 4096, 0.1)
    eager(Xb.to(dev), Wb.to(dev))
    for i in (0, 1, 2, 10, 11, 39):
        X, W = cases[i]
        X.mul_(-1.0)
        y = gc.v9_linear_forward_cuda_graph(X, W)
        assert torch.equal(y, eager(X, W)), f"entry {i} replayed wrong after later captures"
        assert torch.equal(y, -first[i]) or torch.allclose(y.float(), -first[i].float(), atol=1e-2)
    assert gc.cuda_graph_cache_stats()["n_entries"] == 40


def test_v9_linear_cuda_graph_wrapper(small):
    from zip_kernel_b200.v9_linear_graph import V9LinearCudaGraph
    X1, W = small
    m = V9LinearCudaGraph(W, warmup_iters=2)
    for X in (X1, torch.cat([X1, X1 * 2]).contiguous(), X1, (X1 * 3).reshape(1, 1, -1)):
        y = m(X)
        assert y.shape == X.shape[:-1] + (W.d_out,)
        assert torch.equal(y.reshape(-1, W.d_out), eager(X.reshape(-1, W.d_in), W))
    assert m.n_graphs() == 2
    Xl = torch.cat([X1] * 130).contiguous()
    assert torch.equal(m(Xl), eager(Xl, W)) and m.n_graphs() == 2     # many tokens: eager
    with pytest.raises(ValueError):
        m(X1[:, :128])
