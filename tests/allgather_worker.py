"""One rank of the multi-GPU check of the fused all-gather epilogue (run under torchrun by test_allgather_gpu.py)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    from eval_test_b200 import inputs, nvfp4_dual_gemm, nvfp4_gemm, shard
    m, n, k, l = 512, 256 * world, 1024, 2
    full = inputs.gemm_quantized(m, n, k, l, seed=9, device=dev)        # the same seed on every rank
    want = nvfp4_gemm.custom_kernel(full, alpha=0.5).clone()
    out = shard.GatheredOutput(m, n, l, dev)
    out.buf.fill_(float("nan"))
    out.wait_all()                                                     # nobody writes into a buffer still being filled
    shard.gemm_allgather(shard.shard_gemm(full, rank, world), out, rank, alpha=0.5)
    out.wait_all()
    torch.cuda.synchronize()
    assert torch.equal(out.view().view(torch.int16), want.view(torch.int16)), "gemm copy differs"
    fd = inputs.dual_gemm_quantized(m, n, k, 1, seed=10, device=dev)
    wantd = nvfp4_dual_gemm.custom_kernel(fd).clone()
    outd = shard.GatheredOutput(m, n, 1, dev)
    outd.buf.fill_(float("nan"))
    outd.wait_all()
    shard.dual_gemm_allgather(shard.shard_dual_gemm(fd, rank, world), outd, rank)
    outd.wait_all()
    torch.cuda.synchronize()
    assert torch.equal(outd.view().view(torch.int16), wantd.view(torch.int16)), "dual gemm copy differs"
    print("allgather ok", rank, flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
