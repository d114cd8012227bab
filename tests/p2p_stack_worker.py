"""Worker of tests/test_stack_p2p.py: one rank of a 2-GPU column-parallel decode stack (launched by
torch.distributed.run).  Compares the peer-store gathers with the NCCL gather (bit-exact) and with the
1-rank stack (fp16 tolerance) over several steps with fresh inputs, eagerly and from a CUDA graph."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "llm_quantization-kernel_b200"))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from crispybits_kernels.stack import DecodeStack
    kw = dict(n_blocks=3, d_model=1024, d_ff=2048, bitmap=[4, 2, 3], device=dev, std=0.05)
    one = DecodeStack(rank=0, world=1, **kw)
    stacks = {c: DecodeStack(rank=rank, world=world, comm=c, **kw) for c in ("nccl", "p2p", "p2p_barrier", "p2p_seq")}
    g = torch.Generator().manual_seed(5)
    for B in (1, 3, 8):
        for it in range(4):
            x = torch.randn(B, 1024, generator=g).half().to(dev)
            ref = one.step(x).float()
            y = {c: s.step(x).clone() for c, s in stacks.items()}
            torch.cuda.synchronize()
            for c in ("p2p", "p2p_barrier", "p2p_seq"):
                assert torch.equal(y[c], y["nccl"]), (c, B, it)
                assert stacks[c].peer_status() == 0, (c, stacks[c].peer_status())
            err = ((y["nccl"].float() - ref).abs().max() / ref.abs().max()).item()
            assert err < 4e-3, (B, it, err)
    # graph replays keep the launch counts going
    x = torch.randn(2, 1024, generator=g).half().to(dev)
    want = stacks["nccl"].step(x).clone()
    for c in ("p2p", "p2p_barrier", "p2p_seq"):
        st = stacks[c]
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            st.step(x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            y = st.step(x)
        for _ in range(5):
            gr.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, want), c
        assert st.peer_status() == 0
        dist.barrier()
    if rank == 0:
        print("P2P_STACK_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
