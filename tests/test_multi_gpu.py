"""Two NCCL ranks on two GPUs: batch-index sharding of a batched contraction (no collective) and N-column
slabs of one GEMM followed by the optional all-gather, each checked against the unsharded CUDA result bit
for bit and against the CPU oracle within 1e-3.  Skipped on a single-GPU box."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmp):
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from nova_compiler_b200 import ops, sharding
    from oracle import oracle as O
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)  # identical data on every rank
    q = torch.randn(6, 256, 128, device="cuda", generator=g).to(torch.float16)
    k = torch.randn(6, 128, 320, device="cuda", generator=g).to(torch.float16)
    full = ops.batch_matmul(q, k)
    mine, (start, count) = sharding.sharded_batch_matmul(q, k, rank, world)
    ok = torch.equal(mine, full[start:start + count])
    a = (torch.rand(512, 384, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand(384, 1000, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    whole = ops.matmul(a, b)
    slab, (s0, n0) = sharding.slab_matmul(a, b, rank, world)
    ok = ok and torch.equal(slab, whole[:, s0:s0 + n0])
    gathered = sharding.gather_slabs(slab, b.shape[1])
    ok = ok and torch.equal(gathered, whole)
    bits = lambda t: t.contiguous().cpu().view(torch.int16).numpy().view(np.uint16)
    want = O.gemm(bits(a), bits(b), dtype_in="bf16")
    ok = ok and O.rel_fro(O.from_bits(bits(gathered), "bf16"), O.from_bits(want, "bf16")) <= 1e-3
    # the same slabs pushed by the contraction's epilogue into every rank's matrix (no all-gather)
    pm = sharding.PeerMatrix(a.shape[0], b.shape[1] + 24, torch.bfloat16)   # 1024 columns: slabs stay 16-byte aligned
    bw = torch.zeros(384, 1024, device="cuda", dtype=torch.bfloat16)
    bw[:, :1000] = b
    bias = (torch.rand(1024, device="cuda", generator=g) - 0.5).to(torch.bfloat16)
    pm.local.fill_(-3.0)
    torch.cuda.synchronize()
    dist.barrier()
    sharding.slab_matmul_push(a, bw, pm, bias=bias, act="gelu")
    torch.cuda.synchronize()
    dist.barrier()                      # every rank's kernel has completed: the whole matrix is here
    whole_w = ops.linear(a, bw, bias, act="gelu")
    ok = ok and torch.equal(pm.local, whole_w)
    pm.close()
    ok = ok and ops.device_status() == 0
    with open(os.path.join(tmp, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "FAILED")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_batch_and_slab_sharding(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
