"""torchrun worker of tests/test_peer_gather_gpu.py::test_two_processes_over_ipc: one rank per GPU."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    import torch
    import torch.distributed as dist

    import qwen35x_b200 as engine
    from helpers import make_activations, make_weight, to_torch_bf16
    from qwen35x_b200.sharding import PeerGather

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    m, n, k = 512, 2560, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=3)
    x = to_torch_bf16(make_activations(m, k, seed=4))
    a_codes, a_scales, g = engine.quantize_activations(x)
    full = engine.gemm_w4a4(engine.Nvfp4Weight.from_host(codes, scales, s2), a_codes, a_scales, g, m)
    shard = engine.Nvfp4Weight.from_host(codes, scales, s2, shard_index=rank, shard_count=world)
    gather = PeerGather(m, n)
    ok = True
    for _ in range(3):
        gather.tensor().zero_()
        torch.cuda.synchronize()
        dist.barrier()
        c = gather.project(shard, a_codes, a_scales, g)
        torch.cuda.synchronize()
        gather.check()
        ok = ok and bool(torch.equal(c, full))
        dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
