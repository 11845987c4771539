"""One rank of the multi-GPU check of the ttnn tensor-parallel surface (launched by test_ttnn_tp_multi_gpu.py through
torchrun): column-sharded weights, ttnn.linear + ttnn.all_gather (NCCL) against ttnn.linear_all_gather / linear_multi (the
gather in the matmul's epilogue), chained through several layers. Prints 'TP-OK <rank>' on success."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path[:0] = [ROOT, os.path.join(ROOT, "tt-metal_b200"), HERE]

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import ttnn
    mesh = ttnn.open_device_mesh(ttnn.DeviceGrid(1, world), list(range(world)))
    gen = torch.Generator().manual_seed(7)
    H, F = 1024, 2048
    x = torch.randn(1, 1, 32, H, generator=gen).bfloat16()
    layers = []
    for _ in range(3):
        layers.append({k: torch.randn(*shape, generator=gen) * 0.03 for k, shape in
                       (("wq", (H, H)), ("wk", (H, 256)), ("wv", (H, 256)), ("w1", (H, F)), ("w3", (H, F)), ("w2", (F, H)))})
    shard = lambda w: ttnn.from_torch(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=mesh.device,
                                      mesh_mapper=ttnn.ShardTensorToMesh(mesh, dim=-1))
    tt_layers = [{k: shard(w) for k, w in L.items()} for L in layers]
    a0 = ttnn.MultiDeviceTensor(ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=mesh.device), mesh)
    torch.cuda.synchronize()
    dist.barrier()

    def run(fused):
        a = a0
        trace = []
        for L in tt_layers:
            if fused:
                q, k, v = ttnn.linear_multi(a, [L["wq"], L["wk"], L["wv"]], all_gather_first=True)
                h, _ = ttnn.linear_multi(q, [L["w1"], L["w3"]], activation="silu", all_gather_first=True)
                a = ttnn.linear_all_gather(h, L["w2"])
            else:
                q = ttnn.all_gather(ttnn.linear(a, L["wq"]), dim=-1, num_links=1)
                k, v = ttnn.linear(a, L["wk"]), ttnn.linear(a, L["wv"])
                h = ttnn.all_gather(ttnn.linear(q, L["w1"], activation="silu"), dim=-1, num_links=1)
                a = ttnn.all_gather(ttnn.linear(h, L["w2"]), dim=-1, num_links=1)
            trace += [ttnn.to_torch(k).float(), ttnn.to_torch(a).float()]
        return trace

    ref = run(False)
    for rep in range(3):
        got = run(True)
        for r, g in zip(ref, got):
            assert r.shape == g.shape
            num = (r - g).abs().max() / r.abs().max().clamp_min(1e-6)
            assert float(num) <= 2e-2, float(num)      # both paths round to bf16 at every layer; sums may differ in order
    # the gathered activations are identical on every rank
    mine = got[-1].double().sum().reshape(1).cuda()
    both = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    assert all(float(b) == float(mine) for b in both)
    torch.cuda.synchronize()
    dist.barrier()
    print(f"TP-OK {rank}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
