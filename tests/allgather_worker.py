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
    # The whole protocol, three rounds into the SAME buffers with different operands: launch, wait_all, a reader on the
    # stream (a checksum of this rank's copy), release, next launch.  Without release() a rank that is ahead would
    # overwrite a copy whose reader has not run yet; nothing synchronises the host between the rounds.
    rounds, sums = [], []
    for seed in (21, 22, 23):
        d = inputs.gemm_quantized(m, n, k, l, seed=seed, device=dev)
        rounds.append((shard.shard_gemm(d, rank, world), nvfp4_gemm.custom_kernel(d, alpha=0.5).view(torch.int16).clone()))
    torch.cuda.synchronize()
    dist.barrier()
    for sh, _ in rounds:
        shard.gemm_allgather(sh, out, rank, alpha=0.5)
        out.wait_all()
        sums.append(out.view().view(torch.int16).to(torch.int64).sum())     # the reader, stream-ordered
        out.release()
    torch.cuda.synchronize()
    for (_, ref), got in zip(rounds, sums):
        assert int(got) == int(ref.to(torch.int64).sum()), "a copy was overwritten before its reader ran"
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
