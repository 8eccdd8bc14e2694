"""The sequence-sharded protocol on two CPU ranks (gloo): carries, gathers, folds and the
parameter-gradient all-reduce, with the float64 oracle standing in for the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import scan_oracle as O
from tests.helpers import scan_inputs


class OracleOps:
    """Same contracts as mamba_b200.lshard.CudaOps, computed with the float64 CPU oracle."""

    @staticmethod
    def _delta(delta, bias):
        return delta if bias is None else torch.nn.functional.softplus(delta + bias)

    @staticmethod
    def carry_pass(x, delta, A, Bm, Cm, bias, skip_last=0):
        d = OracleOps._delta(delta, bias)
        _, h = O.selective_scan_f64(x, d, A, Bm, Cm, torch.zeros(x.shape[2]), return_last_state=True)
        out = torch.stack([torch.exp(d.double().sum(1).unsqueeze(-1) * A.double()), h])
        if skip_last:                      # the product leaves these rows out of the pass and returns zeros
            out[:, out.shape[1] - skip_last:] = 0
        return out

    @staticmethod
    def fold_range(P_all, S_all, init, first, num, reverse):
        """P_all, S_all: (B, pieces, ED, N) -> (B, num, ED, N): state entering pieces first .. first+num-1."""
        R = P_all.shape[1]
        out = []
        for i in range(first, first + num):
            cur = torch.zeros_like(P_all[:, 0]) if init is None else init.clone()
            for r in (range(R - 1, i, -1) if reverse else range(i)):
                cur = P_all[:, r] * cur + S_all[:, r]
            out.append(cur)
        return torch.stack(out, dim=1)

    @staticmethod
    def full_fwd(x, delta, A, Bm, Cm, D, z, bias, h_in, want_carries):
        y, hT = O.selective_scan_f64(x, OracleOps._delta(delta, bias), A, Bm, Cm, D, z=z, h0=h_in,
                                     return_last_state=True)
        return y, hT, h_in          # the "carries" of the stand-in are just the incoming state

    @staticmethod
    def rev_carry_pass(delta, z, dy, Cm, A, bias, skip_first=0):
        Bsz, L, ED = delta.shape
        h0 = torch.zeros(Bsz, ED, A.shape[1], dtype=torch.float64, requires_grad=True)
        x0 = torch.zeros(Bsz, L, ED, dtype=torch.float64)
        y = O.selective_scan_f64(x0, OracleOps._delta(delta, bias), A, torch.zeros_like(Cm), Cm,
                                 torch.zeros(ED), z=z, h0=h0)
        y.backward(dy.double())
        g = h0.grad
        if skip_first:
            g[:skip_first] = 0
        return g

    @staticmethod
    def full_bwd(x, delta, A, Bm, Cm, D, z, bias, dy, carries, g_in):
        lv = [t.double().clone().requires_grad_() for t in (x, delta, z, Bm, Cm, A, D)]
        xx, dd, zz, BB, CC, AA, DD = lv
        bl = None if bias is None else bias.double().clone().requires_grad_()
        h0 = carries.double().clone().requires_grad_()
        y, hT = O.selective_scan_f64(xx, OracleOps._delta(dd, bl), AA, BB, CC, DD, z=zz, h0=h0,
                                     return_last_state=True)
        ((y * dy.double()).sum() + (hT * g_in).sum()).backward()
        return (xx.grad, dd.grad, zz.grad, BB.grad, CC.grad, AA.grad, DD.grad,
                None if bl is None else bl.grad, h0.grad)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, use_bias, out, S=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mamba_b200 import lshard
        inp = scan_inputs(77, 2, 48, 6, 8, structured_A=False, big_delta=True)
        g = torch.Generator().manual_seed(5)
        bias = (torch.randn(6, generator=g) - 1.0) if use_bias else None
        if use_bias:
            inp["delta"] = torch.randn(2, 48, 6, generator=g)
        Ls = 48 // world
        sl = lambda t: t[:, rank * Ls:(rank + 1) * Ls].double()
        args = (sl(inp["x"]), sl(inp["delta"]), inp["A"].double(), sl(inp["B"]), sl(inp["C"]),
                inp["D"].double(), sl(inp["z"]), None if bias is None else bias.double())
        y, h_in, P_all, carries, hT = lshard.sharded_forward(OracleOps, dist.group.WORLD, *args, subshards=S)
        grads = lshard.sharded_backward(OracleOps, dist.group.WORLD, *args, sl(inp["gy"]), h_in, P_all, subshards=S)
        out[rank] = dict(y=y.detach(), grads=[None if t is None else t.detach() for t in grads])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("use_bias,S", [(False, 1), (True, 1), (True, 3)])
def test_two_cpu_ranks_reproduce_the_single_sequence(use_bias, S):
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.start_processes(_worker, args=(world, _free_port(), use_bias, out, S), nprocs=world, join=True,
                       start_method="spawn")
    # single-sequence answer
    inp = scan_inputs(77, 2, 48, 6, 8, structured_A=False, big_delta=True)
    g = torch.Generator().manual_seed(5)
    bias = (torch.randn(6, generator=g) - 1.0) if use_bias else None
    if use_bias:
        inp["delta"] = torch.randn(2, 48, 6, generator=g)
    lv = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
    bl = None if bias is None else bias.double().requires_grad_()
    dl = lv["delta"] if bl is None else torch.nn.functional.softplus(lv["delta"] + bl)
    y = O.selective_scan_f64(lv["x"], dl, lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"])
    y.backward(inp["gy"].double())
    tol = dict(rtol=1e-9, atol=1e-11)
    ys = torch.cat([out[r]["y"] for r in range(world)], 1)
    assert torch.allclose(ys, y.detach(), **tol)
    for i, k in enumerate(("x", "delta", "z", "B", "C")):
        got = torch.cat([out[r]["grads"][i] for r in range(world)], 1)
        assert torch.allclose(got, lv[k].grad, **tol), k
    for r in range(world):                       # parameter gradients: all-reduced, equal on every rank
        assert torch.allclose(out[r]["grads"][5], lv["A"].grad, **tol)
        assert torch.allclose(out[r]["grads"][6], lv["D"].grad, **tol)
        if bl is not None:
            assert torch.allclose(out[r]["grads"][7], bl.grad, **tol)
    # the carry leaving rank 0 to the left is the gradient w.r.t. a (zero) initial state
    assert out[0]["grads"][8].shape == (2, 6, 8)


def test_one_row_cut_on_one_rank_leaves_out_the_unused_carries():
    """Single rank, single batch row: the forward carry pass leaves out the last piece and the reverse one
    the first piece (nothing consumes their carries); the result must still be the uncut scan."""
    from mamba_b200 import split
    inp = scan_inputs(78, 1, 64, 6, 8, structured_A=False, big_delta=True)
    g = torch.Generator().manual_seed(6)
    bias = torch.randn(6, generator=g) - 1.0
    inp["delta"] = torch.randn(1, 64, 6, generator=g)
    h0 = torch.randn(1, 6, 8, generator=g).double()
    args = (inp["x"].double(), inp["delta"].double(), inp["A"].double(), inp["B"].double(), inp["C"].double(),
            inp["D"].double(), inp["z"].double(), bias.double())
    seen = {}

    class Spy(OracleOps):
        @staticmethod
        def carry_pass(*a, **k):
            seen["fwd"] = k
            return OracleOps.carry_pass(*a, **k)

        @staticmethod
        def rev_carry_pass(*a, **k):
            seen["bwd"] = k
            return OracleOps.rev_carry_pass(*a, **k)

    y, h_in, P_all, carries, hT = split.split_forward(Spy, None, *args, h0=h0, subshards=4)
    grads = split.split_backward(Spy, None, *args, inp["gy"].double(), h_in, P_all, subshards=4)
    assert seen == {"fwd": {"skip_last": 1}, "bwd": {"skip_first": 1}}
    lv = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
    bl = bias.double().requires_grad_()
    h0l = h0.clone().requires_grad_()
    yr, hTr = O.selective_scan_f64(lv["x"], torch.nn.functional.softplus(lv["delta"] + bl), lv["A"], lv["B"], lv["C"],
                                   lv["D"], z=lv["z"], h0=h0l, return_last_state=True)
    yr.backward(inp["gy"].double())
    tol = dict(rtol=1e-9, atol=1e-11)
    assert torch.allclose(y, yr.detach(), **tol) and torch.allclose(hT, hTr.detach(), **tol)
    for i, k in enumerate(("x", "delta", "z", "B", "C", "A", "D")):
        assert torch.allclose(grads[i], lv[k].grad, **tol), k
    assert torch.allclose(grads[7], bl.grad, **tol)
    assert torch.allclose(grads[8], h0l.grad, **tol)


def test_pick_subshards():
    from mamba_b200.lshard import pick_subshards
    assert pick_subshards(8, 2048, 1536, 1) == 1            # already enough rows x channel tiles
    assert pick_subshards(1, 65536, 2048, 1) == 16          # one long row of a 1024-wide model: cut it up
    assert pick_subshards(1, 131072, 5120, 1) == 8          # about two waves of CTAs are enough
    assert pick_subshards(1, 16384, 5120, 8) > 1            # several ranks: the carry passes exist anyway
    assert pick_subshards(1, 40, 5120, 1) == 1              # not divisible into 16-step pieces
    assert pick_subshards(1, 2048, 2048, 1) == 1            # short: the extra launches would eat the gain
    assert pick_subshards(1, 4096, 64, 1) == 8              # pieces stay at least 512 timesteps long
