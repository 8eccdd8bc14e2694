"""Sequence-sharded scan on the GPU: the shard-local kernels (carry pass, decay product, fold,
reverse carry pass) chained on one device, and the real NCCL path when two GPUs are present."""
import os
import socket

import pytest
import torch

from oracle import scan_oracle as O
from tests.helpers import scan_inputs, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL, ATOL = 1e-4, 1e-5


def _emulate(inp, R, dtype, bias=None):
    """Run R shards one after another on one GPU through CudaOps (no collective needed)."""
    from mamba_b200.lshard import CudaOps as K
    c = lambda t: t.to(DEV).to(dtype).contiguous()
    f = lambda t: None if t is None else t.to(DEV).float().contiguous()
    x, dl, z, Bm, Cm, dy = (c(inp[k]) for k in ("x", "delta", "z", "B", "C", "gy"))
    A, D, b = f(inp["A"]), f(inp["D"]), f(bias)
    L = x.shape[1]
    Ls = L // R
    sl = lambda t, r: t[:, r * Ls:(r + 1) * Ls] if r < R - 1 else t[:, r * Ls:]
    SP = [K.carry_pass(sl(x, r), sl(dl, r), A, sl(Bm, r), sl(Cm, r), b) for r in range(R)]
    S = torch.stack([sp[1] for sp in SP], dim=1)                    # (B, R, ED, N): state reached from zero
    P = torch.stack([sp[0] for sp in SP], dim=1)                    # decay product of every shard
    h_in = K.fold_range(P, S, None, 0, R, False)                    # state entering every shard, one launch
    ys, cars = [], []
    for r in range(R):
        y, hT, car = K.full_fwd(sl(x, r), sl(dl, r), A, sl(Bm, r), sl(Cm, r), D, sl(z, r), b, h_in[:, r].contiguous(), True)
        ys.append(y)
        cars.append(car)
    G = torch.stack([K.rev_carry_pass(sl(dl, r), sl(z, r), sl(dy, r), sl(Cm, r), A, b) for r in range(R)], dim=1)
    g_in = K.fold_range(P, G, None, 0, R, True)
    outs = []
    for r in range(R):
        outs.append(K.full_bwd(sl(x, r), sl(dl, r), A, sl(Bm, r), sl(Cm, r), D, sl(z, r), b, sl(dy, r), cars[r],
                               g_in[:, r].contiguous()))
    cat = lambda i: torch.cat([o[i] for o in outs], 1)
    tot = lambda i: sum(o[i] for o in outs)
    return dict(y=torch.cat(ys, 1), x=cat(0), delta=cat(1), z=cat(2), B=cat(3), C=cat(4), A=tot(5), D=tot(6),
                bias=None if b is None else tot(7))


@pytest.mark.parametrize("R,L", [(2, 64), (4, 200), (8, 1024)])
def test_shards_chained_on_one_gpu_match_oracle(R, L):
    inp = scan_inputs(300 + L, 2, L, 40, 16, structured_A=False, big_delta=(L < 500))
    got = _emulate(inp, R, torch.float32)
    lv = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
    y = O.selective_scan_f64(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"])
    y.backward(inp["gy"].double())
    assert_close(got["y"], y.float(), RTOL, ATOL, "y")
    for k in ("x", "delta", "z", "B", "C", "A", "D"):
        scale = lv[k].grad.abs().max().item()
        assert_close(got[k], lv[k].grad.float(), RTOL, max(ATOL, ATOL * scale * 4), f"grad {k}")


def test_sharded_equals_unsharded_kernel_long_bf16():
    """bf16, softplus inside, 8 shards of a 16k sequence against the single launch."""
    import mamba_b200
    inp = scan_inputs(9, 1, 16384, 64, 16, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    bias = torch.randn(64, generator=g) * 0.3 - 4.0
    inp["delta"] = (torch.randn(1, 16384, 64, generator=g) * 0.5).bfloat16().float()
    got = _emulate(inp, 8, torch.bfloat16, bias=bias)
    c = lambda k: inp[k].to(DEV).bfloat16().requires_grad_()
    lv = dict(x=c("x"), delta=c("delta"), z=c("z"), B=c("B"), C=c("C"),
              A=inp["A"].to(DEV).requires_grad_(), D=inp["D"].to(DEV).requires_grad_())
    bl = bias.to(DEV).requires_grad_()
    y = mamba_b200.selective_scan_fn(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"], delta_bias=bl)
    y.backward(inp["gy"].to(DEV).bfloat16())
    assert_close(got["y"], y, 2e-2, 2e-2)
    for k in ("x", "delta", "z"):
        assert_close(got[k], lv[k].grad, 2e-2, 2e-2, k)
    for k in ("B", "C"):
        assert_close(got[k].bfloat16(), lv[k].grad, 2e-2, 5e-2 * lv[k].grad.float().abs().max().item(), k)
    for k, ref in (("A", lv["A"].grad), ("D", lv["D"].grad), ("bias", bl.grad)):
        assert_close(got[k], ref, 1e-3, 1e-3 * ref.abs().max().item(), k)


def test_single_rank_subsharded_matches_oracle():
    """One rank, one long row: the slice is cut into sub-shards scanned as batch rows."""
    import torch.distributed as dist
    from mamba_b200.lshard import selective_scan_lsharded, pick_subshards
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device(DEV))
    try:
        inp = scan_inputs(91, 1, 8192, 64, 16, structured_A=False)
        assert pick_subshards(1, 8192, 64, 1) > 1
        lv = {k: inp[k].to(DEV).requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
        y = selective_scan_lsharded(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"])
        y.backward(inp["gy"].to(DEV))
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()
    ref = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
    yo = O.selective_scan_f64(ref["x"], ref["delta"], ref["A"], ref["B"], ref["C"], ref["D"], z=ref["z"])
    yo.backward(inp["gy"].double())
    assert_close(y, yo.float(), RTOL, ATOL, "y")
    for k in ref:
        scale = ref[k].grad.abs().max().item()
        assert_close(lv[k].grad, ref[k].grad.float(), RTOL, max(ATOL, ATOL * scale * 4), f"grad {k}")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from mamba_b200.lshard import selective_scan_lsharded
        inp = scan_inputs(55, 2, 512, 48, 16, structured_A=False)
        Ls = 512 // world
        dev = torch.device("cuda", rank)
        sl = lambda k: inp[k][:, rank * Ls:(rank + 1) * Ls].to(dev).requires_grad_()
        lv = dict(x=sl("x"), delta=sl("delta"), z=sl("z"), B=sl("B"), C=sl("C"),
                  A=inp["A"].to(dev).requires_grad_(), D=inp["D"].to(dev).requires_grad_())
        y = selective_scan_lsharded(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"])
        y.backward(inp["gy"][:, rank * Ls:(rank + 1) * Ls].to(dev))
        torch.cuda.synchronize()
        out[rank] = dict(y=y.detach().cpu(), **{k: v.grad.cpu() for k, v in lv.items()})
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_nccl_match_oracle():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.start_processes(_nccl_worker, args=(world, _free_port(), out), nprocs=world, join=True, start_method="spawn")
    inp = scan_inputs(55, 2, 512, 48, 16, structured_A=False)
    lv = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
    y = O.selective_scan_f64(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"])
    y.backward(inp["gy"].double())
    assert_close(torch.cat([out[r]["y"] for r in range(world)], 1), y.float(), RTOL, ATOL)
    for k in ("x", "delta", "z", "B", "C"):
        got = torch.cat([out[r][k] for r in range(world)], 1)
        scale = lv[k].grad.abs().max().item()
        assert_close(got, lv[k].grad.float(), RTOL, max(ATOL, ATOL * scale * 4), k)
    for k in ("A", "D"):
        for r in range(world):
            scale = lv[k].grad.abs().max().item()
            assert_close(out[r][k], lv[k].grad.float(), RTOL, max(ATOL, ATOL * scale * 4), k)
