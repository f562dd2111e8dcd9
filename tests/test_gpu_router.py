"""GPU parity, routing: expert indices bit-exact against the oracle (both its operator form and the CPU daemon's form),
weights bit-exact against the operator form and within 2 ulp of the daemon's division form."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


@pytest.mark.parametrize("M,Ex,k,renorm,lbf", [(1, 64, 8, True, True), (16, 512, 10, True, True), (33, 160, 8, False, True),
                                              (7, 1024, 16, True, False), (5, 37, 3, True, False)])
def test_softmax_router_bit_exact(E, oracle, M, Ex, k, renorm, lbf):
    import torch
    rng = np.random.default_rng(M * 1000 + Ex + k)
    lg = rng.normal(0, 1, (M, Ex + 3)).astype(np.float32)        # ld > E: trailing columns are not router logits
    ids, w = E.router_softmax_topk(torch.from_numpy(lg).cuda(), k, renorm, lbf, E=Ex)
    i0, w0 = oracle.router_softmax_topk(lg, k, renorm, lbf, 0, E=Ex)
    assert np.array_equal(ids.cpu().numpy(), i0)
    assert w.cpu().numpy().tobytes() == w0.tobytes()
    i1, w1 = oracle.router_softmax_topk(lg, k, renorm, lbf, 1, E=Ex)
    assert np.array_equal(ids.cpu().numpy(), i1)
    assert np.max(np.abs(w.cpu().numpy() - w1) / w1) < 1e-6


def test_softmax_router_ties(E, oracle):
    import torch
    lg = np.array([[1.0, 3.0, 3.0, -2.0, 3.0, 0.5, 3.0009765625, 1.0], [0.0] * 8], np.float32)
    ids, w = E.router_softmax_topk(torch.from_numpy(lg).cuda(), 3, True, True)
    assert ids.cpu().numpy().tolist() == [[1, 2, 4], [0, 1, 2]]
    ids, _ = E.router_softmax_topk(torch.from_numpy(lg).cuda(), 3, True, False)
    assert ids.cpu().numpy().tolist() == [[6, 1, 2], [0, 1, 2]]
    # bf16-rounded logits make ties common: a whole batch must still agree with the oracle
    rng = np.random.default_rng(11)
    lg = np.round(rng.normal(0, 1, (64, 512)) * 4).astype(np.float32) / 4
    ids, w = E.router_softmax_topk(torch.from_numpy(lg).cuda(), 10, True, True)
    i0, w0 = oracle.router_softmax_topk(lg, 10, True, True, 0)
    assert np.array_equal(ids.cpu().numpy(), i0) and w.cpu().numpy().tobytes() == w0.tobytes()


@pytest.mark.parametrize("M,Ex,k", [(8, 160, 8), (1, 256, 8), (19, 64, 6)])
def test_sigmoid_router_bit_exact(E, oracle, M, Ex, k):
    import torch
    rng = np.random.default_rng(M + Ex)
    lg = rng.normal(0, 1, (M, Ex)).astype(np.float32)
    bias = rng.normal(0, 0.3, Ex).astype(np.float32)
    ids, w = E.router_topk(torch.from_numpy(lg).cuda(), torch.from_numpy(bias).cuda(), k, 2.5)
    i0, w0 = oracle.router_sigmoid_topk(lg, bias, k, 2.5, 0)
    assert np.array_equal(ids.cpu().numpy(), i0) and w.cpu().numpy().tobytes() == w0.tobytes()
    i1, w1 = oracle.router_sigmoid_topk(lg, bias, k, 2.5, 1)
    assert np.array_equal(ids.cpu().numpy(), i1)
    assert np.max(np.abs(w.cpu().numpy() - w1) / w1) < 1e-6
    ids, w = E.router_topk(torch.from_numpy(lg).cuda(), None, k, 1.0)
    i0, w0 = oracle.router_sigmoid_topk(lg, None, k, 1.0, 0)
    assert np.array_equal(ids.cpu().numpy(), i0) and w.cpu().numpy().tobytes() == w0.tobytes()


def test_zipf_biased_routing_matches(E, oracle):
    """Hot-expert skew (N(0,1) logits plus a per-expert Zipf(1.1) log-weight bias): indices still bit-exact."""
    import torch
    rng = np.random.default_rng(12)
    Ex = 160
    zipf = 1.0 / np.arange(1, Ex + 1) ** 1.1
    bias = np.log(zipf / zipf.sum())[rng.permutation(Ex)].astype(np.float32)
    lg = (rng.normal(0, 1, (8, Ex)) + bias).astype(np.float32)
    ids, w = E.router_softmax_topk(torch.from_numpy(lg).cuda(), 8, True, True)
    i0, w0 = oracle.router_softmax_topk(lg, 8, True, True, 0)
    assert np.array_equal(ids.cpu().numpy(), i0) and w.cpu().numpy().tobytes() == w0.tobytes()
