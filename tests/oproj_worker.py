"""Child process of tests/test_gpu_peer.py::test_oproj_sum_between_real_gpus: one rank per GPU, each with its
own columns of the projection weight; the kernel's result (sum over the ranks in its epilogue, residual
added, one rounding) against an fp32 product of the unsharded operands, and the same bits on every rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from pie_b200 import ops  # noqa: E402
from pie_b200 import workloads as W  # noqa: E402
from pie_b200.parallel import PeerReduce  # noqa: E402

STEP = 2.0 ** -7


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo")  # host-side exchange of the handles and barriers only
    dt = torch.bfloat16
    hidden = 2048
    k_full = 1024
    kl = k_full // world
    seed = 0
    for mode in ("fp32", "storage"):
        pr = PeerReduce(1400, hidden, dt, dev, partial_sums=mode)
        # rows: a decode step's few, a ragged tile edge, enough for the wide tiles; several steps each so that the
        # staging, the flags and both output buffers are reused
        cases = ((37, True), (128, False), (300, True), (1400, True), (5, True)) if mode == "fp32" else \
            ((37, True), (1400, False), (300, True))
        for n, with_res in cases:
            for step in range(3):
                seed += 1
                a = W.randn((n, k_full), 100 + seed, dt, 0.5, device=dev)
                w = W.randn((hidden, k_full), 200 + seed, dt, 0.5, device=dev)
                res = W.randn((n, hidden), 300 + seed, dt, 1.0, device=dev) if with_res else None
                a_r = a[:, rank * kl:(rank + 1) * kl]                   # strided views: rows of the full matrices
                w_r = w[:, rank * kl:(rank + 1) * kl]
                got = pr.oproj(a_r, w_r, res)
                torch.cuda.synchronize(dev)
                assert ops.device_error(dev) is None
                want = a.float() @ w.float().t()
                if res is not None:
                    want = want + res.float()
                err = (got.float() - want).abs()
                parts = [a[:, r * kl:(r + 1) * kl].float() @ w[:, r * kl:(r + 1) * kl].float().t() for r in range(world)]
                if mode == "fp32":
                    floor = 0.5 * (k_full ** 0.5) * 0.25
                    tol = STEP * want.abs().clamp_min(floor)
                else:
                    # every partial sum is rounded to 16 bits on its way (2^-9 of ITS size, which can exceed the
                    # sum's), then the result once more
                    tol = 2.0 ** -8 * (want.abs() + sum(x.abs() for x in parts)) + 1e-3
                bad = err > tol
                assert not bool(bad.any()), f"rank {rank} {mode} n {n} step {step}: max err {err.max().item()}"
                if mode == "fp32":
                    # the sum in rank order, every partial an fp32 product: what the kernel adds up (its own
                    # accumulation order inside a partial differs by fp32 rounding only)
                    seq = torch.zeros((n, hidden), dtype=torch.float32, device=dev)
                    for r in range(world):
                        seq = seq + parts[r]
                    if res is not None:
                        seq = seq + res.float()
                    flips = (got != seq.to(dt)).float().mean().item()
                    assert flips < 0.02, f"rank {rank} n {n}: {flips:.4f} of the elements round differently"
                sums = [None] * world
                dist.all_gather_object(sums, int(got.view(torch.int16).to(torch.int64).sum().item()))
                assert len(set(sums)) == 1, sums
        pr.close()
    print("OPROJ-OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
