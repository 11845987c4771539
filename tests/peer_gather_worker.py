"""One rank of the multi-GPU check of ttb_matmul_peer (launched by test_peer_gather_multi_gpu.py through torchrun).

Every rank holds column shard `rank` of each weight, runs the gathering matmul, then a consuming matmul that waits for
the gather point, and compares both with fp32 torch matmuls of the unpacked weights. Prints 'PEER-OK <rank>' on success."""
import ctypes
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path[:0] = [ROOT, os.path.join(ROOT, "tt-metal_b200"), HERE]

import torch
import torch.distributed as dist

import cabi


def pcc(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.corrcoef(torch.stack([a, b]))[0, 1])


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from ttnn.peer import GatherRing
    lib = cabi.load()
    M = 32
    shapes = [(4096, 1024), (8192, 256), (1024, 3584), (2048, 128)]            # (K, N per rank)
    ring = GatherRing(rank, world, max(world * M * N * 2 for _, N in shapes), slots=2)
    gen = torch.Generator(device="cuda").manual_seed(1234)                        # same stream of numbers on every rank
    for step in range(3):
        for K, N in shapes:
            x = torch.randn(M, K, generator=gen, device="cuda").bfloat16()
            w_all = torch.randn(K, world * N, generator=gen, device="cuda") * 0.02
            K2, N2 = world * N, 256
            w2 = torch.randn(K2, N2, generator=gen, device="cuda") * 0.02
            shard = w_all[:, rank * N:(rank + 1) * N].contiguous()
            wp = lib.pack(shard, cabi.BFLOAT8_B, 1, K, N)
            w2p = lib.pack(w2, cabi.BFLOAT8_B, 1, K2, N2)
            w_all_q = torch.cat([lib.unpack(lib.pack(w_all[:, r * N:(r + 1) * N].contiguous(), cabi.BFLOAT8_B, 1, K, N), cabi.BFLOAT8_B, 1, K, N)
                                 .reshape(K, N) for r in range(world)], dim=1)
            w2_q = lib.unpack(w2p, cabi.BFLOAT8_B, 1, K2, N2).reshape(K2, N2)
            a = lib.tilize(x, 1, M, K)
            nb = lib.matmul_peer_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, N)
            ws = torch.zeros(nb, dtype=torch.uint8, device="cuda")
            nb2 = lib.matmul_peer_workspace_bytes(cabi.BFLOAT8_B, 1, M, K2, N2)
            ws2 = torch.zeros(nb2, dtype=torch.uint8, device="cuda")
            y2 = torch.empty(M * N2, dtype=torch.bfloat16, device="cuda")
            torch.cuda.synchronize()
            dist.barrier()                                  # keeps the ranks' launches close in time
            slot = ring.take(world * M * N * 2)
            flags = cabi.MM_WORKSPACE_ZEROED | cabi.MM_WEIGHTS_RESIDENT
            lib.check(lib.cdll.ttb_matmul_peer(a.data_ptr(), cabi.BFLOAT16, wp.data_ptr(), cabi.BFLOAT8_B, None, None, cabi.BFLOAT16, 1, M, K, N,
                                               0, flags, ws.data_ptr(), nb, ctypes.byref(ring.gather(slot)), None, None))
            lib.check(lib.cdll.ttb_matmul_peer(ring.out_ptr(slot), cabi.BFLOAT16, w2p.data_ptr(), cabi.BFLOAT8_B, None, y2.data_ptr(),
                                               cabi.BFLOAT16, 1, M, K2, N2, 0, flags, ws2.data_ptr(), nb2, None,
                                               ctypes.byref(ring.wait(slot)), None))
            lib.check(lib.check_status(None))
            gathered = torch.empty(M * K2, dtype=torch.bfloat16, device="cuda")
            lib.check(lib.cdll.ttb_memcpy_d2d(gathered.data_ptr(), ring.out_ptr(slot), M * K2 * 2, None))
            torch.cuda.synchronize()
            y = lib.untilize(gathered, 1, M, K2).reshape(M, K2).float()
            y_ref = x.float() @ w_all_q
            rel = float((y - y_ref).abs().max() / y_ref.abs().max())
            assert pcc(y, y_ref) >= 0.9999 and rel <= 1e-2, (step, K, N, pcc(y, y_ref), rel)
            z = lib.untilize(y2, 1, M, N2).reshape(M, N2).float()
            z_ref = y @ w2_q
            rel2 = float((z - z_ref).abs().max() / z_ref.abs().max())
            assert pcc(z, z_ref) >= 0.9999 and rel2 <= 1e-2, (step, K, N, "consumer", pcc(z, z_ref), rel2)
            # every rank holds the same bytes
            mine = gathered.view(torch.int16).to(torch.int64).sum().reshape(1)
            both = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(both, mine)
            assert all(int(b) == int(mine) for b in both)
    torch.cuda.synchronize()
    dist.barrier()
    print(f"PEER-OK {rank}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
