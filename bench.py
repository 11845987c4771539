"""Benchmark of the block-float weight-matmul path on B200.

Workload (all N): the Llama-2-70B decode weight matmuls, batch 32, 80 layers, every weight bfloat8_b packed from
N(0, 0.02), column-sharded over the N GPUs, with the four per-layer output all-gathers (NCCL) of the tensor-parallel
scheme. One "step" = one pass over all 80 layers = 32 generated tokens. Strong scaling: the model is fixed, each
GPU streams 1/N of the weight bytes.

  python bench.py [--gpus N] [--steps K] [--warmup W]            # this framework
  python bench.py --impl reference ...                            # the reference's CPU path on the host cores
  torchrun ... bench.py --gpus N ...                              # N > 1: one rank per GPU

Prints one JSON line (rank 0). `value` is tokens/s with everything resident in HBM, the whole step replayed as one
CUDA graph; `e2e` is the same step driven through the public ttnn API with host activations copied in and the
result copied out every step; `roofline` is the achieved weight-streaming bandwidth of the matmul kernel.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tt-metal_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

BATCH, HIDDEN, KV, FFN, LAYERS = 32, 8192, 1024, 28672, 80
BF16, F32, BFP8, BFP4 = 0, 1, 3, 4
TILE_BYTES = {BFP8: 1088, BFP4: 576}
METRIC = "decode weight-GEMM tok/s (Llama-2-70B, bfloat8_b weights, batch 32)"
WORKLOAD = ("llama2-70b tensor-parallel decode weight matmuls: batch 32, hidden 8192, kv 1024, ffn 28672, 80 layers, "
            "bfloat8_b weights column-sharded over the GPUs, 4 output all-gathers per layer")


def layer_gemms(G):
    """(name, K, N per GPU, gather output?) for one Llama-2-70B decoder layer's weight matmuls."""
    return [("wq", HIDDEN, HIDDEN // G, True), ("wk", HIDDEN, KV // G, False), ("wv", HIDDEN, KV // G, False),
            ("wo", HIDDEN, HIDDEN // G, True), ("w1", HIDDEN, FFN // G, True), ("w3", HIDDEN, FFN // G, False),
            ("w2", FFN, HIDDEN // G, True)]


class Workload:
    """A sweep of `layers` identical groups of weight matmuls: gemms = [(name, K, N, weight format, gather?)]."""

    def __init__(self, key, G):
        self.key = key
        self.rows = BATCH
        if key == "c5":
            self.metric, self.unit, self.text = METRIC, "tok/s", WORKLOAD
            self.layers = LAYERS
            self.gemms = [(n, K, N, BFP8, g) for n, K, N, g in layer_gemms(G)]
            self.seed = 4
        elif key == "c3":
            self.metric, self.unit = "decode weight-GEMM tok/s (Mistral-7B sweep, batch 32)", "tok/s"
            self.text = ("mistral-7b decode weight-matmul sweep: batch 32, hidden 4096, 32 layers; Wq/Wo 4096x4096, Wk/Wv 4096x1024, "
                         "w2 14336x4096 in bfloat8_b, w1/w3 4096x14336 in bfloat4_b")
            self.layers = 32
            self.gemms = [("wq", 4096, 4096, BFP8, False), ("wk", 4096, 1024, BFP8, False), ("wv", 4096, 1024, BFP8, False),
                          ("wo", 4096, 4096, BFP8, False), ("w1", 4096, 14336, BFP4, False), ("w3", 4096, 14336, BFP4, False),
                          ("w2", 14336, 4096, BFP8, False)]
            self.seed = 2
        elif key == "c2":
            self.metric, self.unit = "bfp8_b GEMM HBM GB/s (Falcon-7B h_to_4h decode linear)", "GB/s"
            self.text = ("single decode ttnn.linear, Falcon-7B h_to_4h: activation bf16 [32, 4544], weight bfloat8_b [4544, 18176]; "
                         "4 distinct weights used in rotation so that no launch finds its weight in L2")
            self.layers = 4
            self.gemms = [("h_to_4h", 4544, 18176, BFP8, False)]
            self.seed = 1
        elif key == "c4":
            self.metric, self.unit = "prefill GEMM bf16 TFLOP/s (Llama-2-70B MLP shape, bfloat8_b weight)", "TFLOP/s"
            self.text = ("prefill matmul, Llama-2-70B MLP shape: activation bf16 [2048, 8192] x weight bfloat8_b [8192, 28672], fp32 "
                         "accumulate, bf16 output; 2 distinct weights used in rotation")
            self.layers = 2
            self.rows = 2048
            self.gemms = [("w1", 8192, 28672, BFP8, False)]
            self.seed = 3
        else:
            raise SystemExit(f"unknown workload {key}")
        if key != "c5" and G != 1:
            raise SystemExit(f"workload {key} is a single-GPU configuration")

    def bytes_per_layer(self):
        """Algorithmic bytes: packed weight + bf16 activations read + bf16 outputs written."""
        return sum(K * N // 1024 * TILE_BYTES[f] + self.rows * K * 2 + self.rows * N * 2 for _, K, N, f, _ in self.gemms)

    def flops_per_layer(self):
        return sum(2 * self.rows * K * N for _, K, N, _, _ in self.gemms)

    def weight_bytes_per_layer(self):
        return sum(K * N // 1024 * TILE_BYTES[f] for _, K, N, f, _ in self.gemms)


def peaks(key="hbm_gbs"):
    """Roofline denominators measured on this pool's B200s (driver-written file), else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)[key]), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}[key], "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, enabled=True):
        self.index, self.rows, self.proc, self.enabled = index, [], None, enabled

    def __enter__(self):
        if not self.enabled:      # only the rank that prints the line samples (several nvidia-smi at once slow each other down)
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def mark(self, name):
        """Remembers the wall-clock time of `name` ("start" / "end" of the timed region)."""
        setattr(self, "t_" + name, time.time())

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, window=None):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t0, t1 = window if window else (getattr(self, "t_start", 0.0), getattr(self, "t_end", float("inf")))
        inside = [r for t, r in self.rows if t0 <= t <= t1 + 0.02]
        # a timed region shorter than a few sampling periods: add the samples of the identical replays that ran right
        # before and after it (same graph, same load)
        t2 = getattr(self, "t_end_load", t1)
        if window:
            rows = inside
        else:
            rows = inside if len(inside) >= 3 else [r for t, r in self.rows if getattr(self, "t_load", 0.0) <= t <= t2 + 0.02]
        for r in rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "window": "timed region" if len(inside) >= 3 else "timed region + identical replays around it"}


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own path for this workload = host bfloat8_b packing + fp32 torch matmul on the unpacked
# weights (the golden its tests compare against), timed on the host cores on a bounded sample.
def cpu_reference_sample(threads=None):
    import numpy as np
    import torch
    import oracle
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    ref = oracle.ref()
    impl, kind = (ref, "reference") if ref is not None else (oracle.port(), "port")
    g = torch.Generator().manual_seed(4)
    # packing sample: the Wk weight of one layer (8192 x 1024), the reference's from_torch sequence, one thread
    wk = (torch.randn(HIDDEN, KV, generator=g) * 0.02).numpy()
    t0 = time.perf_counter()
    packed = impl.from_torch(wk, oracle.BFP8_B, 1, HIDDEN, KV)
    t_pack = time.perf_counter() - t0
    pack_gbs = (wk.nbytes + packed.nbytes) / t_pack / 1e9
    # matmul sample: one full decoder layer (G = 1) in fp32 on unpacked weights
    x_h = torch.randn(BATCH, HIDDEN, generator=g).bfloat16().float()
    x_f = torch.randn(BATCH, FFN, generator=g).bfloat16().float()
    weights = []
    w_small = torch.from_numpy(impl.to_torch(packed, oracle.BFP8_B, 1, HIDDEN, KV).reshape(HIDDEN, KV).copy())
    for _, K, N, _ in layer_gemms(1):
        # tile the unpacked sample weight to the layer's shapes: values stay bfloat8_b-representable N(0, 0.02)
        weights.append(w_small.repeat(-(-K // HIDDEN), -(-N // KV))[:K, :N].contiguous())

    def one_layer():
        s = 0.0
        for (name, K, N, _), w in zip(layer_gemms(1), weights):
            y = torch.matmul(x_f if K == FFN else x_h, w)
            s += float(y[0, 0])
        return s
    return one_layer, threads, kind, t_pack, pack_gbs


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    one_layer, threads, kind, t_pack, pack_gbs = cpu_reference_sample()
    for _ in range(max(args.warmup, 1)):
        one_layer()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        one_layer()
        times.append(time.perf_counter() - t0)
    t_layer = sum(times) / len(times)
    t_step = t_layer * LAYERS
    value = BATCH / t_step
    sample = (f"one decoder layer (7 fp32 torch matmuls on unpacked bfloat8_b weights) per step, scaled x{LAYERS}; "
              f"host packing of one 8192x1024 weight took {t_pack:.2f} s ({pack_gbs:.3f} GB/s, 1 thread)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"tp{args.gpus}"},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# Ratio of DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum of one profiler capture) to algorithmic bytes of the
# dominant kernels; the captures and their commands are summarised under profiles/.
DECODE_KERNEL = "matmul_decode_tmem_kernel"
DECODE_TRAFFIC_RATIO = 90.92 / 89.21
DECODE_TRAFFIC_SOURCE = "profiles/matmul_decode_tmem_c2_falcon_h_to_4h.md"
PREFILL_TRAFFIC_RATIO = 525.5 / 400.6


class _DeviceView:
    """Zero-copy torch view of raw device memory through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def load_lib():
    path = os.path.join(ROOT, "tt-metal_b200", "lib", "libttb.so")
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build the extension first (python -c 'import __graft_entry__ as g; g.build()')")
    lib = ctypes.CDLL(path)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.ttb_last_error.restype = ctypes.c_char_p
    lib.ttb_pack_bfp.argtypes = [vp, i32, vp, i32, i64, i64, i64, i32, i32, vp]
    lib.ttb_tilize.argtypes = [vp, vp, i32, i64, i64, i64, vp]
    lib.ttb_untilize.argtypes = [vp, vp, i32, i64, i64, i64, vp]
    lib.ttb_unpack_bfp.argtypes = [vp, i32, vp, i32, i64, i64, i64, i32, i32, vp]
    lib.ttb_matmul_workspace_bytes.argtypes = [i32, i64, i64, i64, i64, i32]
    lib.ttb_matmul_workspace_bytes.restype = i64
    lib.ttb_matmul.argtypes = [vp, i32, vp, i32, vp, vp, i32, i64, i64, i64, i64, i32, i32, vp, i64, vp]
    lib.ttb_check_status.argtypes = [vp]
    lib.ttb_matmul_peer_workspace_bytes.argtypes = [i32, i64, i64, i64, i64]
    lib.ttb_matmul_peer_workspace_bytes.restype = i64
    lib.ttb_matmul_peer.argtypes = [vp, i32, vp, i32, vp, vp, i32, i64, i64, i64, i64, i32, i32, vp, i64, vp, vp, vp]
    lib.ttb_matmul_multi_workspace_bytes.argtypes = [i32, i64, i64, i64, i32, vp]
    lib.ttb_matmul_multi_workspace_bytes.restype = i64
    lib.ttb_matmul_multi.argtypes = [vp, i32, i32, vp, i32, vp, vp, i32, i64, i64, i64, vp, i32, i32, vp, i64, vp, vp, vp]
    return lib


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run for N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU implementation of the product path")
    torch.cuda.set_device(local_rank)
    torch.backends.cuda.matmul.allow_tf32 = False      # the parity block's fp32 reference is a true fp32 matmul
    dev_t = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev_t)
    G = world
    lib = load_lib()

    def ck(rc):
        if rc != 0:
            raise RuntimeError(lib.ttb_last_error().decode())

    ZEROED = 8 | (0 if args.no_overlap else 64)   # workspace head is zero; weights are long resident (overlapped launches)
    import ttnn
    device = ttnn.open_device(local_rank)
    mesh = ttnn.open_device_mesh(ttnn.DeviceGrid(1, G), list(range(G))) if G > 1 else None

    def barrier():
        if G > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def tilize(x):
        out = torch.empty(x.numel(), dtype=x.dtype, device=dev_t)
        ck(lib.ttb_tilize(x.data_ptr(), out.data_ptr(), x.element_size(), 1, x.shape[0], x.shape[1], None))
        return out

    def untilize(t, rows, cols):
        out = torch.empty(rows * cols, dtype=t.dtype, device=dev_t)
        ck(lib.ttb_untilize(t.data_ptr(), out.data_ptr(), t.element_size(), 1, rows, cols, None))
        return out.reshape(rows, cols)

    def unpack(p, fmt, K, N):
        out = torch.empty(K * N, dtype=torch.float32, device=dev_t)
        ck(lib.ttb_unpack_bfp(p.data_ptr(), fmt, out.data_ptr(), F32, 1, K, N, 1, 0, None))
        return out.reshape(K, N)

    def pcc_and_rel(y, ref):
        y, ref = y.float().reshape(-1), ref.float().reshape(-1)
        ym, rm = y - y.mean(), ref - ref.mean()
        pcc = float((ym * rm).sum() / (ym.norm() * rm.norm()).clamp_min(1e-30))
        rel = float((y - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        return pcc, rel

    # ============================================================================================================
    def time_workload(wl, steps, warmup, clocks):
        """Builds the workload's weights on the device, captures one step as a CUDA graph and times `steps` replays.
        Returns the measurements and the state the end-to-end and parity legs reuse."""
        gen = torch.Generator(device=dev_t).manual_seed(wl.seed + 1000 * rank)
        gemms, NLAYERS, ROWS = wl.gemms, wl.layers, wl.rows
        weights = []          # [layer][gemm] -> packed uint8 tensor: distinct per layer, generated and packed on the device
        t_setup = time.perf_counter()
        for _ in range(NLAYERS):
            row = []
            for _, K, N, fmt, _ in gemms:
                w = torch.randn(K, N, generator=gen, device=dev_t, dtype=torch.float32) * 0.02
                p = torch.empty(K * N // 1024 * TILE_BYTES[fmt], dtype=torch.uint8, device=dev_t)
                ck(lib.ttb_pack_bfp(w.data_ptr(), F32, p.data_ptr(), fmt, 1, K, N, 1, 0, None))
                row.append(p)
                del w
            weights.append(row)
        torch.cuda.synchronize()
        t_setup = time.perf_counter() - t_setup

        acts = {}             # K -> (host bf16 [rows, K], tiled device copy): a fresh N(0,1) activation per distinct K
        for _, K, _, _, _ in gemms:
            if K not in acts:
                x = torch.randn(ROWS, K, generator=torch.Generator().manual_seed(40 + len(acts))).bfloat16()
                acts[K] = (x, tilize(x.to(dev_t)))
        outs = [torch.empty(ROWS * N, dtype=torch.bfloat16, device=dev_t) for _, _, N, _, _ in gemms]
        gathered = [torch.empty(G * ROWS * N, dtype=torch.bfloat16, device=dev_t) if g else None for _, _, N, _, g in gemms]
        ws_bytes = max(lib.ttb_matmul_workspace_bytes(f, 1, ROWS, K, N, 0) for _, K, N, f, _ in gemms)
        # Tensor parallel: the all-gather is the matmul's epilogue (peer stores over NVLink into every rank's copy) unless
        # --gather nccl asks for a separate NCCL all-gather after the matmul.
        ring = None
        if G > 1 and args.gather == "fused":
            from ttnn.peer import GatherRing
            ring = GatherRing(rank, G, max(G * ROWS * N * 2 for _, _, N, _, g in gemms if g), slots=4)
            assert (NLAYERS * sum(1 for x in gemms if x[4])) % ring.slots == 0
        # Launch groups: matmuls of a layer that multiply the same activation go out as one launch (q/k/v; w1/w3), unless
        # --no-group asks for one launch per weight. Only the first weight of a group is ever gathered.
        SHARE = {"wq": "qkv", "wk": "qkv", "wv": "qkv", "w1": "w13", "w3": "w13"}
        groups = []
        for i, (name, K, N, fmt, g) in enumerate(gemms):
            key = None if args.no_group else SHARE.get(name)
            if key is not None and groups and groups[-1][0] == key and len(groups[-1][1]) < 4 and not g:
                groups[-1][1].append(i)
            else:
                groups.append((key, [i]))
        groups = [idxs for _, idxs in groups]
        arrays = {}
        for idxs in groups:
            arr_n = (ctypes.c_int64 * len(idxs))(*[gemms[i][2] for i in idxs])
            if ROWS <= 256:
                ws_bytes = max(ws_bytes, lib.ttb_matmul_multi_workspace_bytes(gemms[idxs[0]][3], 1, ROWS, gemms[idxs[0]][1], len(idxs), arr_n))
        ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device=dev_t)

        def group_arrays(layer, idxs):
            key = (layer, idxs[0])
            if key not in arrays:
                n = len(idxs)
                arrays[key] = ((ctypes.c_void_p * n)(*[weights[layer][i].data_ptr() for i in idxs]),
                               (ctypes.c_void_p * n)(*[outs[i].data_ptr() for i in idxs]),
                               (ctypes.c_int64 * n)(*[gemms[i][2] for i in idxs]))
            return arrays[key]

        def launch_group(layer, idxs, stream_handle, fused, pending, flags=ZEROED):
            """One launch of a layer's group; returns the gather point the next launch has to wait for (or None)."""
            _, K, N, fmt, g = gemms[idxs[0]]
            arr_w, arr_o, arr_n = group_arrays(layer, idxs)
            if ROWS > 256:      # prefill shape: the single-weight entry point (tensor-bound kernel)
                ck(lib.ttb_matmul(acts[K][1].data_ptr(), BF16, weights[layer][idxs[0]].data_ptr(), fmt, None, outs[idxs[0]].data_ptr(),
                                  BF16, 1, ROWS, K, N, 0, flags, ws.data_ptr(), ws_bytes, stream_handle))
                return None
            slot = ring.take(G * ROWS * N * 2) if (fused and g) else None
            ck(lib.ttb_matmul_multi(acts[K][1].data_ptr(), BF16, len(idxs), arr_w, fmt, None, arr_o, BF16, 1, ROWS, K, arr_n,
                                    0, flags, ws.data_ptr(), ws_bytes,
                                    ctypes.byref(ring.gather(slot)) if slot is not None else None,
                                    ctypes.byref(ring.wait(pending)) if pending is not None else None, stream_handle))
            return slot

        def sweep(stream_handle, with_gather=True):
            fused = ring is not None and with_gather
            pending = None          # gather point whose result the next launch has to wait for
            for layer in range(NLAYERS):
                for idxs in groups:
                    pending = launch_group(layer, idxs, stream_handle, fused, pending)
                    if gemms[idxs[0]][4] and G > 1 and with_gather and not fused:
                        # tiled [32, N/G] shards are whole tile runs: the rank-major gather is the tiled [32, N] tensor
                        dist.all_gather_into_tensor(gathered[idxs[0]], outs[idxs[0]])
            if pending is not None:
                ring.stream_wait(pending, stream_handle)     # the step ends when this rank holds every gathered result

        def capture(with_gather):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                sweep(side.cuda_stream, with_gather)      # warm-up outside capture (lazy module loading, NCCL channels)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            ck(lib.ttb_check_status(None))                 # a kernel whose bounded wait ran out ends the run here, not after K steps
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                sweep(torch.cuda.current_stream().cuda_stream, with_gather)
            return graph

        def keep_load_while(cond, graph, seconds=3.0):
            """Replays the graph (untimed) while rank 0's `cond()` holds (at most `seconds`), the same number of times on every rank."""
            t_stop = time.time() + seconds
            while True:
                flag = torch.tensor([1 if (rank == 0 and cond() and time.time() < t_stop) else 0], device=dev_t)
                if G > 1:
                    dist.broadcast(flag, 0)
                if int(flag.item()) == 0:
                    break
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize()

        def timed_replays(graph, nsteps, nwarm, sampler=None):
            if sampler:
                sampler.mark("load")
            for _ in range(nwarm):
                graph.replay()
            if sampler:
                keep_load_while(lambda: len(sampler.rows) == 0, graph)       # nvidia-smi takes a moment to deliver its first sample
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if sampler:
                sampler.mark("start")
            e0.record()
            for _ in range(nsteps):
                graph.replay()
            e1.record()
            barrier()
            if sampler:
                sampler.mark("end")
                # a timed region shorter than three sampling periods: keep the identical load running until three samples exist
                keep_load_while(lambda: sum(1 for t, _ in sampler.rows if t >= sampler.t_start) < 3, graph)
                sampler.mark("end_load")
            ms = e0.elapsed_time(e1)
            if G > 1:
                t = torch.tensor([ms], device=dev_t)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
            return ms

        graph_full = capture(True)      # also gives nvidia-smi time to start sampling
        ms_step = timed_replays(graph_full, steps, warmup, clocks) / steps
        clock_summary = clocks.summary() if clocks else None
        # ---- roofline of the dominant kernel: the matmul-only sweep (no collectives, no peer stores), same weights ------
        graph_mm = None
        if G > 1:
            graph_mm = capture(False)
            ms_mm = timed_replays(graph_mm, steps, 1) / steps
        else:
            ms_mm = ms_step
        ck(lib.ttb_check_status(None))
        R = argparse.Namespace(wl=wl, weights=weights, acts=acts, outs=outs, gathered=gathered, groups=groups, gemms=gemms, ring=ring,
                               ws=ws, ws_bytes=ws_bytes, ms_step=ms_step, ms_mm=ms_mm, t_setup=t_setup, clocks=clock_summary,
                               launch_group=launch_group, graphs=[graph_full, graph_mm])
        R.launches_per_step = NLAYERS * len(groups)
        R.bytes_per_step = wl.bytes_per_layer() * NLAYERS
        R.flops_per_step = wl.flops_per_layer() * NLAYERS
        R.tensor_bound = wl.unit == "TFLOP/s"
        if wl.unit == "tok/s":
            R.to_value = lambda sec: BATCH / sec
        elif wl.unit == "TFLOP/s":
            R.to_value = lambda sec: R.flops_per_step / sec / 1e12
        else:
            R.to_value = lambda sec: R.bytes_per_step / sec / 1e9
        R.value = R.to_value(ms_step * 1e-3)
        if R.tensor_bound:
            R.achieved = R.flops_per_step / (ms_mm * 1e-3) / 1e12
            R.peak, R.peak_kind = peaks("bf16_tflops")
        else:
            R.achieved = R.bytes_per_step / (ms_mm * 1e-3) / 1e9
            R.peak, R.peak_kind = peaks("hbm_gbs")
        return R

    # ============================================================================================================
    def parity_block(R):
        """Outside the timed region: layer 0's launches once more, every output compared with an fp32 matmul of the
        unpacked weight shards (torch.cat over the ranks for gathered outputs). With the fused gather the gathered bytes are
        also compared with the NCCL form (the same launch without the gather epilogue, then an NCCL all-gather) and across
        ranks; both launches add their split-K partial sums in a fixed order (TTB_MM_DETERMINISTIC), so equal means equal bytes."""
        FIXED = 8 | 32      # workspace head is zero; deterministic reduction order
        wl, gemms, ROWS = R.wl, R.gemms, R.wl.rows
        fused = R.ring is not None
        worst_pcc, worst_rel, checked = 1.0, 0.0, 0
        equal_ranks, equal_nccl = True, True
        pending = None
        for idxs in R.groups:
            K, fmt, g = gemms[idxs[0]][1], gemms[idxs[0]][3], gemms[idxs[0]][4]
            slot = R.launch_group(0, idxs, None, fused, pending, FIXED)
            pending = None
            if slot is not None:
                R.ring.stream_wait(slot)
            torch.cuda.synchronize()
            ck(lib.ttb_check_status(None))
            x = R.acts[K][0].to(dev_t).float()
            for j, i in enumerate(idxs):
                N = gemms[i][2]
                w_ref = unpack(R.weights[0][i], fmt, K, N)
                if ROWS > 512:      # prefill-sized: a seeded sample of rows keeps the fp32 reference cheap
                    rows_idx = torch.randperm(ROWS, generator=torch.Generator().manual_seed(7))[:256].to(dev_t)
                else:
                    rows_idx = None
                ref = (x if rows_idx is None else x[rows_idx]) @ w_ref
                del w_ref
                if g and G > 1 and j == 0:
                    parts = [torch.empty_like(ref) for _ in range(G)]
                    dist.all_gather(parts, ref.contiguous())
                    ref = torch.cat(parts, dim=1)
                    if fused:
                        nbytes = G * ROWS * N * 2
                        got_t = torch.as_tensor(_DeviceView(R.ring.out_ptr(slot), nbytes), device=dev_t).view(torch.bfloat16).clone()
                        # the same result by the NCCL form: the same launch into local outputs, then an all-gather of the tiled
                        # shard (a run of whole tiles, so the rank-major gather is the tiled [rows, G*N] tensor), byte for byte
                        R.launch_group(0, idxs, None, False, None, FIXED)
                        dist.all_gather_into_tensor(R.gathered[i], R.outs[i])
                        torch.cuda.synchronize()
                        equal_nccl = equal_nccl and bool(torch.equal(got_t, R.gathered[i]))
                    else:
                        dist.all_gather_into_tensor(R.gathered[i], R.outs[i])
                        got_t = R.gathered[i]
                    digest = got_t.view(torch.int16).to(torch.int64).sum().reshape(1)
                    digests = [torch.empty_like(digest) for _ in range(G)]
                    dist.all_gather(digests, digest)
                    equal_ranks = equal_ranks and all(int(d) == int(digests[0]) for d in digests)
                    y = untilize(got_t, ROWS, G * N)
                else:
                    y = untilize(R.outs[i], ROWS, N)
                    if rows_idx is not None:
                        y = y[rows_idx]
                pcc, rel = pcc_and_rel(y, ref)
                worst_pcc, worst_rel, checked = min(worst_pcc, pcc), max(worst_rel, rel), checked + 1
        out = {"pcc": worst_pcc, "max_rel": worst_rel, "outputs_checked": checked, "pass": bool(worst_pcc >= 0.9999 and worst_rel <= 1e-2),
               "vs": "fp32 torch matmul of unpacked shards" + (", torch.cat over ranks" if G > 1 else ""),
               "tolerance": "pcc >= 0.9999 and max|y - ref| / max|ref| <= 1e-2"}
        if G > 1:
            t = torch.tensor([worst_pcc, -worst_rel, 1.0 if equal_ranks else 0.0, 1.0 if equal_nccl else 0.0], device=dev_t, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            out.update({"pcc": float(t[0]), "max_rel": float(-t[1]), "gathered_equal_on_all_ranks": bool(t[2] > 0.5),
                        "pass": bool(t[0] >= 0.9999 and -t[1] <= 1e-2 and t[2] > 0.5 and t[3] > 0.5)})
            if fused:
                out["fused_gather_equals_nccl_gather"] = bool(t[3] > 0.5)
        return out

    # ============================================================================================================
    def time_conversion(fmt, direction, clocks):
        """C1: fp32 [1,1,4096,4096] N(0, 0.02) seed 0 -> packed tiles (or back), device to device, four buffers in rotation
        (256 MB of sources: no launch finds its input in L2)."""
        H = W = 4096
        g0 = torch.Generator(device=dev_t).manual_seed(0)
        srcs = [torch.randn(H, W, generator=g0, device=dev_t) * 0.02 for _ in range(4)]
        packed = [torch.empty(H * W // 1024 * TILE_BYTES[fmt], dtype=torch.uint8, device=dev_t) for _ in range(4)]
        for s_, p_ in zip(srcs, packed):
            ck(lib.ttb_pack_bfp(s_.data_ptr(), F32, p_.data_ptr(), fmt, 1, H, W, 1, 0, None))
        outs_ = [torch.empty(H * W, dtype=torch.float32, device=dev_t) for _ in range(4)] if direction == "unpack" else None
        torch.cuda.synchronize()

        def one(i, st):
            if direction == "pack":
                ck(lib.ttb_pack_bfp(srcs[i % 4].data_ptr(), F32, packed[i % 4].data_ptr(), fmt, 1, H, W, 1, 0, st))
            else:
                ck(lib.ttb_unpack_bfp(packed[i % 4].data_ptr(), fmt, outs_[i % 4].data_ptr(), F32, 1, H, W, 1, 0, st))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        per_graph = 20
        with torch.cuda.graph(graph, stream=side):
            for i in range(per_graph):
                one(i, torch.cuda.current_stream().cuda_stream)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        reps = 400
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        us = e0.elapsed_time(e1) * 1e3 / (reps * per_graph)
        nbytes = H * W * 4 + packed[0].numel()
        peak, kind = peaks("hbm_gbs")
        gbs = nbytes / us / 1e3
        return {"value": gbs, "unit": "GB/s", "us_per_launch": us, "algorithmic_bytes": nbytes, "frac": gbs / peak, "peak_kind": kind,
                "clocks": clocks.summary((t0, t1)) if clocks else None}

    def summarise(R, window_clocks=None):
        return {"value": R.value, "unit": R.wl.unit, "ms_per_step": R.ms_step, "achieved": R.achieved,
                "achieved_unit": "TFLOP/s" if R.tensor_bound else "GB/s", "frac": R.achieved / R.peak, "peak_kind": R.peak_kind,
                "avg_launch_us": R.ms_mm * 1e3 / R.launches_per_step, "clocks": window_clocks or R.clocks}

    # ============================================================================================================
    if args.workload == "c1":
        # C1 on its own: tensor conversion (ttnn.from_torch's pack, ttnn.to_torch's unpack) in both block-float formats;
        # the headline is bfloat8_b packing, `e2e` the same through ttnn.from_torch with the host copy inside.
        if G != 1:
            raise SystemExit("workload c1 is a single-GPU configuration")
        with ClockSampler(local_rank, enabled=True) as clocks:
            conv = {f"{d}_{n}": time_conversion(f, d, clocks) for f, n in ((BFP8, "bfp8"), (BFP4, "bfp4")) for d in ("pack", "unpack")}
            host = (torch.randn(4096, 4096, generator=torch.Generator().manual_seed(0)) * 0.02).pin_memory()
            for _ in range(3):
                t = ttnn.from_torch(host, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                t = ttnn.from_torch(host, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
            torch.cuda.synchronize()
            e2e_s = (time.perf_counter() - t0) / args.steps
        head = conv["pack_bfp8"]
        print(json.dumps({
            "metric": "bfloat8_b pack GB/s (ttnn.from_torch of fp32 [1,1,4096,4096], TILE_LAYOUT)", "value": head["value"], "unit": "GB/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["us_per_launch"] / 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "tensor conversion: fp32 [1,1,4096,4096] N(0, 0.02) -> bfloat8_b tiles, four source buffers in rotation (256 MB, larger than L2)",
                       "timed": "CUDA-graph replay of 20 launches x 400"},
            "clocks": head["clocks"],
            "e2e": {"value": head["algorithmic_bytes"] / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4096 * 4096 * 4, "d2h_bytes_per_step": 0,
                    "ms_per_step": e2e_s * 1e3, "api": "ttnn.from_torch(pinned fp32, dtype=bfloat8_b, layout=TILE_LAYOUT, device)"},
            "gpu_launches": 20 * 400,
            "roofline": {"bound": "hbm", "achieved": head["value"], "peak": head["value"] / head["frac"], "unit": "GB/s", "frac": head["frac"],
                         "traffic": None, "peak_kind": head["peak_kind"], "kernel": "pack_rowmajor_kernel"},
            "extra": conv}), flush=True)
        return

    with ClockSampler(local_rank, enabled=(rank == 0)) as clocks:
        wl = Workload(args.workload, G)
        R = time_workload(wl, args.steps, args.warmup, clocks)
        NLAYERS, ROWS, gemms, groups, weights, acts = wl.layers, wl.rows, R.gemms, R.groups, R.weights, R.acts

        # ---- end to end through the public API: host activations in, result out, every step -------------------------
        def wrap(t_uint8, K, N, fmt):
            return ttnn._ttnn.wrap_device_memory(t_uint8.data_ptr(), ttnn.Shape([K, N]), ttnn.bfloat8_b if fmt == BFP8 else ttnn.bfloat4_b,
                                                 ttnn.TILE_LAYOUT, device)
        tt_weights = [[wrap(weights[l][i], K, N, f) for i, (_, K, N, f, _) in enumerate(gemms)] for l in range(NLAYERS)]
        pinned = {K: v[0].pin_memory() for K, v in acts.items()}
        h2d = sum(p.numel() * 2 for p in pinned.values())
        last_n = gemms[-1][2] * (G if gemms[-1][4] else 1)
        d2h = ROWS * last_n * 2
        fused_api = mesh is not None and args.gather == "fused"

        def e2e_step():
            a = {K: ttnn.from_torch(p, layout=ttnn.TILE_LAYOUT, device=device) for K, p in pinned.items()}
            if mesh is not None:
                a = {K: ttnn.MultiDeviceTensor(t, mesh) for K, t in a.items()}
            y = None
            for layer in range(NLAYERS):
                for idxs in groups:
                    _, K, N, _, g = gemms[idxs[0]]
                    if ROWS <= 256 and (len(idxs) > 1 or (fused_api and g)):
                        # one launch for the weights that share this activation; the first result gathered by the kernel itself
                        y = ttnn.linear_multi(a[K], [tt_weights[layer][i] for i in idxs], all_gather_first=bool(fused_api and g))[0]
                    else:
                        y = ttnn.linear(a[K], tt_weights[layer][idxs[0]])
                    if g and mesh is not None and not fused_api:
                        y = ttnn.all_gather(y, dim=-1, num_links=1)
            return ttnn.to_torch(y)

        for _ in range(min(args.warmup, 3)):
            res = e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            res = e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - t0) / args.steps
        if G > 1:
            t = torch.tensor([e2e_s], device=dev_t, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = t.item()
        assert res.shape == (ROWS, last_n) and bool(torch.isfinite(res.float()).all())

        parity = parity_block(R)

        # DRAM bytes per launch of the dominant kernel, from one profiler capture (dram__bytes_read.sum + dram__bytes_write.sum)
        # of the same kernel, scaled by the bytes a launch covers: the decode kernel moved DECODE_TRAFFIC_RATIO times its
        # algorithmic bytes on the Falcon h_to_4h linear (every weight byte is read once, so traffic grows with the weight);
        # the prefill kernel PREFILL_TRAFFIC_RATIO times on the Llama MLP prefill linear.
        alg_per_launch = R.bytes_per_step / R.launches_per_step
        if R.tensor_bound:
            traffic, traffic_src = alg_per_launch * PREFILL_TRAFFIC_RATIO, "profiles/matmul_prefill_c4_llama70b_mlp.md (same launch)"
        else:
            traffic, traffic_src = alg_per_launch * DECODE_TRAFFIC_RATIO, DECODE_TRAFFIC_SOURCE + ", scaled x(bytes per launch)"
        line = {
            "metric": wl.metric, "value": R.value, "unit": wl.unit, "n_gpus": G, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": R.ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": wl.text, "parallelism": f"tp{G}", "gather": ("none" if G == 1 else args.gather),
                       "launch_groups": [[gemms[i][0] for i in idxs] for idxs in groups], "l2": "per-step working set (%.1f GB per GPU) far exceeds the 126 MB L2" % (R.bytes_per_step / 1e9),
                       "timed": "CUDA-graph replay of the whole step", "setup_s": round(R.t_setup, 2)},
            "clocks": R.clocks,
            "e2e": {"value": R.to_value(e2e_s), "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3,
                    "api": ("ttnn.from_torch -> ttnn.linear_multi / ttnn.linear x%d%s -> ttnn.to_torch" %
                            (NLAYERS * len(groups), "" if mesh is None else (", gather in the matmul epilogue" if fused_api else " + ttnn.all_gather")))},
            "gpu_launches": (R.launches_per_step * (3 if R.tensor_bound else 1) + (1 if R.ring is not None else 0)) * args.steps,   # prefill: re-layout + main + tail launch; fused gather: the step's closing wait kernel
            "roofline": {"bound": "tensor" if R.tensor_bound else "hbm", "achieved": R.achieved, "peak": R.peak,
                         "unit": "TFLOP/s" if R.tensor_bound else "GB/s", "frac": R.achieved / R.peak,
                         "traffic": traffic, "traffic_unit": "bytes per launch", "traffic_source": traffic_src, "peak_kind": R.peak_kind,
                         "kernel": "matmul_prefill_kernel" if R.tensor_bound else DECODE_KERNEL,
                         "launches_per_step": R.launches_per_step, "algorithmic_bytes_per_step": R.bytes_per_step,
                         "avg_launch_us": R.ms_mm * 1e3 / R.launches_per_step},
            "parity": parity,
            "matmul_only_ms": R.ms_mm, "gather_exposed_ms": max(R.ms_step - R.ms_mm, 0.0) if G > 1 else 0.0,
        }

        # ---- the other configurations, measured after the headline in the same process (1 GPU, default workload) ------
        if G == 1 and wl.key == "c5" and not args.no_extra:
            extra = {}
            del tt_weights, weights, acts, res
            R.graphs.clear()
            R = None
            torch.cuda.empty_cache()
            for fmt, fname in ((BFP8, "bfp8"), (BFP4, "bfp4")):
                for direction in ("pack", "unpack"):
                    extra[f"c1_{direction}_{fname}"] = time_conversion(fmt, direction, clocks if rank == 0 else None)
            for key, nsteps in (("c2", 200), ("c3", 20), ("c4", 20)):
                t0 = time.time()
                Rx = time_workload(Workload(key, 1), nsteps, 3, None)
                px = parity_block(Rx)
                entry = summarise(Rx, clocks.summary((t0, time.time())))
                entry["parity"] = {k: px[k] for k in ("pcc", "max_rel", "pass", "outputs_checked")}
                entry["workload"] = Rx.wl.text
                extra[key] = entry
                Rx.graphs.clear()
                del Rx
                torch.cuda.empty_cache()
            line["extra"] = extra

    if rank == 0:
        if G == 1 and not args.no_cpu_baseline and wl.key == "c5":
            one_layer, threads, kind, t_pack, pack_gbs = cpu_reference_sample()
            one_layer()
            t0 = time.perf_counter()
            reps = 3
            for _ in range(reps):
                one_layer()
            t_layer = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {"value": BATCH / (t_layer * LAYERS), "unit": "tok/s", "cores": threads, "kind": kind,
                                    "sample": f"{reps} passes over one decoder layer of fp32 torch matmuls on unpacked weights, scaled x{LAYERS}; "
                                              f"host bfloat8_b packing of one 8192x1024 weight: {t_pack:.2f} s = {pack_gbs:.3f} GB/s on 1 thread"}
        print(json.dumps(line), flush=True)
    if G > 1:
        # Release the captured graphs (they hold NCCL kernels) before the communicator goes away, then leave without the
        # interpreter's teardown: destroying a communicator that captured graphs still reference can block forever.
        if R is not None:
            R.graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: all-gather in the matmul epilogue over peer memory (default) or a separate NCCL all-gather")
    ap.add_argument("--no-group", action="store_true", help="one launch per weight instead of one per group of weights that share an activation")
    ap.add_argument("--no-extra", action="store_true", help="skip the C1-C4 measurements that follow the headline at 1 GPU")
    ap.add_argument("--no-overlap", action="store_true", help="launch every matmul after the previous one has fully completed")
    ap.add_argument("--workload", default="c5", choices=["c5", "c4", "c3", "c2", "c1"],
                    help="c5 = Llama-2-70B TP decode sweep (default, the headline), c4 = Llama-2-70B MLP prefill matmul, "
                         "c3 = Mistral-7B sweep, c2 = Falcon-7B decode linear, c1 = tensor conversion")
    ap.add_argument("--max-seconds", type=int, default=1500, help="watchdog: the process exits with status 3 after this long")
    args = ap.parse_args()

    def _watchdog():
        time.sleep(args.max_seconds)
        sys.stderr.write(f"bench.py: watchdog fired after {args.max_seconds} s\n")
        sys.stderr.flush()
        os._exit(3)
    threading.Thread(target=_watchdog, daemon=True).start()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
