"""Expert-parallel MoE decode through the peer-memory exchange, with the ranks run ONE AFTER THE OTHER on a single GPU
(kernels of different ranks never wait on each other inside one device: every rank's partial is in place before any
combine is launched).  Checks the sliced shared expert, the exchange buffers / flags / epoch parity, the rank-ordered
combine and the bounded flag wait against the oracle and against the single-GPU launch."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from test_moe_gpu import MoeCase, dev, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


@pytest.fixture()
def enc():
    from macseek_b200.core import Enc
    return Enc()


def table_of(case, n_exp):
    return torch.tensor([[s.gate.data_ptr(), s.up.data_ptr(), s.down.data_ptr()] for s in case.slots[:n_exp]],
                        dtype=torch.int64, device="cuda")


@pytest.mark.parametrize("world", (1, 2, 4, 8))
@pytest.mark.parametrize("sh", (ol.Q8_0, ol.Q6_K), ids=["Q8_0", "Q6_K"])
def test_ep_exchange_matches_single_gpu(orc, enc, world, sh):
    from macseek_b200 import ep, quant as q
    n_exp = 16
    case = MoeCase(4096, 2048, ol.IQ1_S, ol.IQ2_XXS, sh, 8, True, n_experts=n_exp)
    table = table_of(case, n_exp)
    comms = ep.EpComm.local(case.D, world)
    try:
        # two exchanges in a row (the slot / flag parity flips), different routings, one of them leaving ranks idle
        for ids in (np.array([13, 2, 7, 8, 0, 15, 5, 10], dtype=np.int32), np.array([0, 1, 2, 3, 4, 5, 6, 7], dtype=np.int32)):
            ids_d = dev(ids)
            keep, h, y, ymag, hmag = case.reference(orc, ids=ids)
            per = n_exp // world
            for r in range(world):
                a = case.args(ids=ids)
                a.y = None
                lo, hi = ep.shared_range(case.I, world, r)
                q.encode_moe_decode_ep(enc, a, table, ids_d, r * per, (r + 1) * per, lo, hi, comms[r])
            outs = []
            for r in range(world):
                hr = dev(case.y0)
                ep.encode_combine(enc, comms[r], hr)
                outs.append(hr)
            enc.wait()
            got = [o.cpu().numpy() for o in outs]
            for r in range(1, world):
                assert np.array_equal(bits(got[r]), bits(got[0])), "ranks disagree"
            assert orc.max_norm_err(got[0], y, ymag) <= 5e-5
    finally:
        for c in comms:
            c.close()


def test_ep_sliced_shared_expert_accumulates_like_the_whole(orc, enc):
    # comm = None: each slice's partial is accumulated into y; the slices together are the whole shared expert
    from macseek_b200 import ep, quant as q
    n_exp = 8
    case = MoeCase(2048, 1024, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 4, True, n_experts=n_exp)
    table = table_of(case, n_exp)
    ids = np.array([5, 1, 6, 2], dtype=np.int32)
    ids_d = dev(ids)
    keep, h, y, ymag, hmag = case.reference(orc, ids=ids)
    a = case.args(ids=ids)
    for r in range(4):
        lo, hi = ep.shared_range(case.I, 4, r)
        q.encode_moe_decode_ep(enc, a, table, ids_d, r * 2, (r + 1) * 2, lo, hi, None)
    enc.wait()
    assert orc.max_norm_err(a.y.cpu().numpy(), y, ymag) <= 5e-5


def test_shared_range_covers_inter():
    from macseek_b200 import ep
    for inter, world in ((2048, 1), (2048, 2), (2048, 8), (2304, 4), (2304, 8), (512, 8)):
        r = [ep.shared_range(inter, world, k) for k in range(world)]
        assert r[0][0] == 0 and r[-1][1] == inter
        assert all(r[k][1] == r[k + 1][0] for k in range(world - 1))
        assert all(lo % 256 == 0 and hi % 256 == 0 and lo <= hi for lo, hi in r)


def test_ep_combine_wait_expires_with_status_3(enc):
    # rank 1 never contributes: rank 0's combine gives up after its (shortened) wait, records status 3 and leaves h alone;
    # msb_device_status() reports it once and the library keeps working afterwards
    from macseek_b200 import _lib, ep, quant as q
    case = MoeCase(1024, 512, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 2, True, n_experts=4)
    table = table_of(case, 4)
    ids_d = dev(np.array([0, 3], dtype=np.int32))
    comms = ep.EpComm.local(case.D, 2)
    _lib.lib.msb_set_peer_wait_cycles(4_000_000)          # ~2 ms
    try:
        a = case.args(ids=[0, 3])
        a.y = None
        q.encode_moe_decode_ep(enc, a, table, ids_d, 0, 2, 0, 256, comms[0])
        h0 = dev(case.y0)
        ep.encode_combine(enc, comms[0], h0)
        enc.stream.synchronize()
        assert _lib.device_status() == 3
        assert _lib.device_status() == 0
        assert np.array_equal(bits(h0.cpu().numpy()), bits(case.y0))
    finally:
        _lib.lib.msb_set_peer_wait_cycles(0)
        for c in comms:
            c.close()
    # a fresh exchange works
    comms = ep.EpComm.local(case.D, 1)
    try:
        a = case.args(ids=[0, 3])
        a.y = None
        q.encode_moe_decode_ep(enc, a, table, ids_d, 0, 4, 0, case.I, comms[0])
        h0 = dev(case.y0)
        ep.encode_combine(enc, comms[0], h0)
        enc.wait()
        assert np.isfinite(h0.cpu().numpy()).all() and not np.array_equal(bits(h0.cpu().numpy()), bits(case.y0))
    finally:
        comms[0].close()

