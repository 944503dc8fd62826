#!/usr/bin/env python
"""Benchmark of the hot path: fp32 GEMM forward + backward (C = A.B, dA = dC.B^T, dB = A^T.dC).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--size 8192] [--impl reference]

One "step" is one forward+backward pass (three GEMMs, transposed operands as stride views) over one
set of seeded synthetic matrices, N(0,1), row-major.  With N > 1 (launched by torch.distributed.run,
one process per GPU) every rank runs its own replica of the step -- the standalone GEMM has no
cross-GPU dependency -- and the reported value is the sum over ranks (weak scaling).

The one JSON line printed by rank 0 carries:
  value      device-resident throughput, 6*M*N*K flop per step, CUDA-event timed, max over ranks
  e2e        the same step through the host-facing call: inputs in pinned host memory, H2D copies,
             the three GEMMs, D2H of the three results, all inside the timed region
  roofline   the tcgen05 GEMM kernel alone (event pairs recorded around each launch by the library)
             against the measured tensor peak: TF32 runs at half the measured bf16 rate and 3xTF32
             spends three tensor-core products per fp32 product, so peak = bf16 / 2 / 3
  cpu_baseline   the CPU oracle (restated tenmo CPU path) on this host's cores, on a bounded sample
--impl reference times that CPU path alone (the reference is Mojo and cannot be built here, so the
oracle port is the reference arm).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fp32_gemm_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def host_isa() -> str:
    """What the CPU baseline's code can use: the oracle is built for AVX2 + FMA (one build runs on every host); the
    host's widest vector extension is named beside it."""
    try:
        with open("/proc/cpuinfo") as f:
            flags = next((line.split(":", 1)[1].split() for line in f if line.startswith("flags")), [])
    except OSError:
        flags = []
    widest = "AVX-512" if "avx512f" in flags else "AVX2" if "avx2" in flags else "unknown"
    return f"built for AVX2+FMA, host has {widest}"


# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one-pass ncu captures of this file's own
# workloads.  A number taken under a profiler is never timed here; only the byte counts are carried over.
NCU_TRAFFIC_BYTES = {
    ("gemm_tc_kernel", 8192): 8.96e9,
    ("colsum_split_kernel", 8192 * 4096): 134.6e6,
    ("ew_kernel<relu_bwd>", 8192 * 4096): 370.8e6,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(source="measured", hbm_gbs=d["hbm_gbs"], bf16_burst=d["bf16_tflops"],
                    bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0)


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle port, bounded sample
# ---------------------------------------------------------------------------------------------------
def cpu_fwd_bwd(size: int, threads: int, seed: int = 0) -> float:
    """Seconds for one forward+backward at size^3 through the oracle (stride views for the transposes)."""
    import numpy as np

    from oracle import ref

    rng = np.random.default_rng(seed)
    A, B, dC = (rng.standard_normal((size, size), np.float32) for _ in range(3))
    Av, Bv, dCv = ref.View.of(A), ref.View.of(B), ref.View.of(dC)
    t0 = time.perf_counter()
    ref.matmul(Av, Bv, threads=threads)
    ref.matmul(dCv, Bv.t(), threads=threads)  # dA = dC.B^T: B^T is a stride view -> the scalar path, as in the reference
    ref.matmul(Av.t(), dCv, threads=threads)  # dB = A^T.dC
    return time.perf_counter() - t0


def cpu_baseline(budget_s: float = 20.0):
    threads = host_cores()
    size = 512
    secs = cpu_fwd_bwd(size, threads)
    # grow the sample while the next size is predicted to stay inside the budget (work grows 8x per doubling)
    while size < 4096 and secs * 8 < budget_s:
        size *= 2
        secs = cpu_fwd_bwd(size, threads)
    flops = 6.0 * size ** 3
    return dict(value=flops / secs / 1e12, unit=UNIT, cores=threads, kind="port",
                sample=f"one fwd+bwd at {size}^3 ({secs:.2f} s), oracle port of matmul_cpu.mojo, {threads} threads over row tiles; "
                       f"{host_isa()}")


def gemm_workload_text(S: int) -> str:
    return (f"fp32 GEMM fwd+bwd (C=A.B, dA=dC.B^T, dB=A^T.dC) at M=N=K={S}, N(0,1) seeded, "
            f"transposes as stride views; 3xTF32: each input split into its lo plane once per step")


def run_reference_arm(args):
    """The reference's own CPU path (oracle port of matmul_cpu.mojo: the Mojo reference cannot be built here) on all
    host threads.  Each step is one fwd+bwd at the requested size when the whole run is predicted to end within
    --ref-budget seconds, else at the largest power-of-two size that does (TFLOP/s is a rate: the sample stands in
    for the full size and the workload text says so)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_cores()
    cpu_fwd_bwd(512, threads)                                   # loads the oracle
    probe = min(2048, args.size)                                # enough row tiles to occupy every thread
    rate = 6.0 * probe ** 3 / cpu_fwd_bwd(probe, threads)      # flop/s, to predict the time of a step
    runs = args.steps + args.warmup
    size = args.size
    if args.ref_size:
        size = args.ref_size
    else:
        while size > 512 and 6.0 * size ** 3 / rate * runs > args.ref_budget:
            size //= 2
        size = 1 << (size.bit_length() - 1) if size != args.size else size
    for _ in range(args.warmup):
        cpu_fwd_bwd(size, threads)
    t0 = time.perf_counter()
    for s in range(args.steps):
        cpu_fwd_bwd(size, threads, seed=s)
    dt = time.perf_counter() - t0
    flops = 6.0 * size ** 3 * args.steps
    value = flops / dt / 1e12
    sample = (f"each step = one fwd+bwd at {size}^3 on {threads} host threads (oracle port; the Mojo reference cannot be built "
              f"here); {host_isa()}")
    workload = gemm_workload_text(args.size)
    if size != args.size:
        workload += f" [CPU arm: timed at {size}^3, extrapolated to {args.size}^3 as a rate]"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "size": args.size, "sample_size": size},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ---------------------------------------------------------------------------------------------------
# clocks sampler
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_first(self, timeout=3.0):
        t0 = time.time()
        while self.proc and not self.lines and time.time() - t0 < timeout:
            time.sleep(0.02)

    def stop(self, t_begin=None, t_end=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in self.lines:
            if t_begin is not None and not (t_begin <= ts <= t_end + 0.1):
                continue  # keep only samples taken while the timed region ran
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# MLP training legs (secondary figures on the same JSON line)
# ---------------------------------------------------------------------------------------------------
def measure_mlps(h, rank, world, local_rank, timed, args):
    """wide_mlp: 4096-4096-4096-4096-1000, global batch 8192 split by rows over the ranks (strong scaling),
    one NCCL sum all-reduce of the flat gradient bucket per step, SGD momentum 0.9.
    mnist_mlp (1 GPU only): 784-128-32-10, batch 64, the step replayed as a CUDA graph (latency-bound:
    samples/s and us/step, no roofline claim)."""
    import numpy as np
    import torch

    from tenmo_b200.parallel import exchange_unique_id, shard_rows, torch_broadcast_bytes
    from tenmo_b200.trainer import MLPTrainer

    out = {}
    legs = set(args.legs.split(","))
    rng = np.random.default_rng(4321)  # same stream on every rank: identical replicas
    gen = torch.Generator(device="cpu").manual_seed(777)

    def uniform_init(dims, limit_fn):
        return ([rng.uniform(-1, 1, (dims[i], dims[i + 1])).astype(np.float32) * np.float32(limit_fn(dims[i], dims[i + 1]))
                 for i in range(len(dims) - 1)], [np.zeros(d, np.float32) for d in dims[1:]])

    if "wide_mlp" in legs:
        out["wide_mlp"] = measure_wide_mlp(h, rank, world, local_rank, timed, args, uniform_init, gen)
    if "cnn" in legs:
        out["cnn"] = measure_cnn(h, rank, world, local_rank, timed, args, rng, gen)
    if "mnist_mlp" in legs and world == 1:
        measure_mnist_mlp.no_cpu = args.no_cpu
        out["mnist_mlp"] = measure_mnist_mlp(h, local_rank, timed, uniform_init, gen)
    return out


def measure_other_sizes(h, algo, timed):
    """The other sizes of the GEMM configuration (square 1024 / 2048 / 4096, skinny 65536 x 784 x 128): forward +
    backward through the plain tenmo_gemm_f32 call, device-resident, a few steps each.  Secondary figures; the
    headline is the largest square size."""
    import torch

    from tenmo_b200 import make_mat

    res = {}
    for name, (M, K, N) in (("1024", (1024,) * 3), ("2048", (2048,) * 3), ("4096", (4096,) * 3), ("skinny_65536x784x128", (65536, 784, 128))):
        A, B, dC = torch.randn(M, K, device="cuda"), torch.randn(K, N, device="cuda"), torch.randn(M, N, device="cuda")
        C, dA, dB = torch.empty(M, N, device="cuda"), torch.empty(M, K, device="cuda"), torch.empty(K, N, device="cuda")
        mA, mB, mdC = (make_mat(t.data_ptr(), tuple(t.shape), (t.shape[1], 1)) for t in (A, B, dC))
        mBt, mAt = make_mat(B.data_ptr(), (N, K), (1, N)), make_mat(A.data_ptr(), (K, M), (1, K))

        def step():
            h.gemm(M, N, K, mA, mB, C.data_ptr(), algo=algo)
            h.gemm(M, K, N, mdC, mBt, dA.data_ptr(), algo=algo)
            h.gemm(K, N, M, mAt, mdC, dB.data_ptr(), algo=algo)

        for _ in range(3):
            step()
        steps = 10
        ms = timed(step, steps)
        res[name] = {"tflops": 6.0 * M * N * K * steps / (ms * 1e-3) / 1e12, "ms_per_step": ms / steps}
        del A, B, dC, C, dA, dB
    torch.cuda.empty_cache()
    return res


def build_with_fallback(build, exchange, uid, h, rank, world, dev):
    """Build a trainer with the requested gradient exchange.  The peer-memory exchange needs CUDA IPC between the
    ranks' processes; where that is refused, every rank falls back to the NCCL exchange together (both run on the GPU)."""
    import torch
    import torch.distributed as dist

    from tenmo_b200 import TenmoError
    from tenmo_b200.parallel import exchange_unique_id, torch_broadcast_bytes

    if world == 1 or exchange == "nccl":
        return build(exchange, uid)
    tr, ok = None, 1
    try:
        tr = build(exchange, None)
    except TenmoError as e:
        ok = 0
        print(f"rank {rank}: peer-memory exchange unavailable ({e}); using NCCL", file=sys.stderr, flush=True)
    flag = torch.tensor([ok], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 1:
        return tr
    if tr is not None:
        tr.close()
    try:
        h.dp_p2p_close()
    except TenmoError:
        pass
    uid = exchange_unique_id(h.dp_get_unique_id, rank, world, torch_broadcast_bytes(dev))
    return build("nccl", uid)


def measure_wide_mlp(h, rank, world, local_rank, timed, args, uniform_init, gen):
    import numpy as np
    import torch

    from tenmo_b200.parallel import exchange_unique_id, shard_rows, torch_all_gather_bytes, torch_broadcast_bytes
    from tenmo_b200.trainer import MLPTrainer

    torch.cuda.nvtx.range_push("wide_mlp")
    dims, gb = [4096, 4096, 4096, 4096, 1000], 8192
    Ws, bs = uniform_init(dims, lambda i, o: np.sqrt(6.0 / i))  # "Kaiming-uniform": U(+-sqrt(6/in))
    lo, hi = shard_rows(gb, rank, world)
    dev = torch.device("cuda", local_rank)
    uid = exchange_unique_id(h.dp_get_unique_id, rank, world, torch_broadcast_bytes(dev)) if args.dp_exchange == "nccl" else None
    def build(exchange, unique_id):
        return MLPTrainer(Ws, bs, batch=hi - lo, lr=0.01, momentum=0.9, algo="3xtf32", handle=h, rank=rank, world=world,
                          unique_id=unique_id, device=local_rank, exchange=exchange, all_gather_bytes=torch_all_gather_bytes(dev),
                          overlap=False if args.dp_no_overlap else (True if args.dp_overlap else None))

    tr = build_with_fallback(build, args.dp_exchange, uid, h, rank, world, dev)
    Xg = torch.randn(gb, dims[0], generator=gen)
    yg = torch.randint(0, dims[-1], (gb,), generator=gen)
    Xh, yh = Xg[lo:hi].contiguous().pin_memory(), yg[lo:hi].contiguous().pin_memory()
    tr.load_batch(Xh, yh)
    for _ in range(3):
        tr.step()
    # The same three steps from the same weights on the same global batch at every N: the loss of the third step
    # (mean over the ranks) and a checksum of the updated parameters make the data-parallel runs comparable.
    check = training_check(tr, world, dev)
    ms = timed(tr.step, args.mlp_steps)
    h.check_device_status()

    loss_host = torch.zeros(args.mlp_steps + 1, dtype=torch.float32).pin_memory()
    e2e_i = [0]

    def e2e_step():
        tr.load_batch(Xh, yh)   # H2D of this rank's rows from pinned memory, on the copy stream, into the idle input set
        tr.step()
        loss_host[e2e_i[0] % loss_host.numel():e2e_i[0] % loss_host.numel() + 1].copy_(tr.loss, non_blocking=True)  # D2H of the loss
        e2e_i[0] += 1

    e2e_step()
    ms_e2e = timed(e2e_step, args.mlp_steps)
    h.check_device_status()
    flops = sum(2.0 * gb * dims[l] * dims[l + 1] * (3 if l > 0 else 2) for l in range(4))
    res = {
        "metric": "mlp_train_samples_per_s", "value": gb * args.mlp_steps / (ms * 1e-3), "unit": "samples/s",
        "ms_per_step": ms / args.mlp_steps, "tflops": flops * args.mlp_steps / (ms * 1e-3) / 1e12, "scaling": "strong",
        "global_batch": gb, "per_rank_batch": hi - lo, "allreduce_bytes_per_step": 0 if world == 1 else tr.numel * 4,
        "e2e_value": gb * args.mlp_steps / (ms_e2e * 1e-3), "e2e_ms_per_step": ms_e2e / args.mlp_steps,
        "e2e_h2d_bytes_per_step": int(Xh.numel() * 4 + yh.numel() * 8) * world, "e2e_d2h_bytes_per_step": 4 * world,
        "steps": args.mlp_steps, "check_after_3_steps": check,
        "config": "4096-4096-4096-4096-1000 Linear+ReLU, softmax-CE, fp32 (3xTF32 GEMMs), N(0,1) inputs, U(+-sqrt(6/in)) weights",
    }
    res["exchange"] = tr.exchange
    res["overlap"] = tr.overlap
    if world > 1 and tr.exchange in ("p2p", "p2p_allreduce"):
        res["exchange_kernel"] = measure_exchange_kernel(tr, h, timed, world)
    if rank == 0 and world == 1 and not args.no_cpu:
        res["cpu_baseline"] = cpu_mlp_baseline(dims, Ws, bs, Xg[:512].numpy(), yg[:512].numpy(), steps=2,
                                               note="wide MLP, a 512-row sample of the 8192-row batch")
    if world > 1:
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier()
        tr.close()
        dist.barrier()
    del tr
    torch.cuda.empty_cache()
    torch.cuda.nvtx.range_pop()
    return res


def measure_exchange_kernel(tr, h, timed, world):
    """The peer-memory exchange kernel alone on the largest layer (nothing else running), against NVLink: per call a rank
    receives (W-1)/W of the range twice -- the peers' gradient copies it reads for its shard and the finished elements the
    peers push into its bucket -- so the inbound traffic per rank is 2 (W-1)/W 4 count bytes (and as much goes out); the
    measured peer-copy bandwidth of this pool is 770 GB/s per direction."""
    import torch

    start, count = max(tr.layer_span, key=lambda sc: sc[1])
    h.set_stream(torch.cuda.current_stream().cuda_stream)

    def call():
        if tr.sharded:   # lr = 0, momentum = 0: parameters and velocities come out as they went in
            h.dp_p2p_sgd_step(start, tr.numel + start, count, tr.V.data_ptr() + 4 * start, 0, 0, 0.0, 0.0, 0.0, 1.0 / world)
        else:
            h.dp_p2p_allreduce_sum(start, count)

    tr.G.zero_()
    for _ in range(3):
        call()
    iters = 10
    ms = timed(call, iters) / iters
    inbound = 2.0 * (world - 1) / world * 4.0 * count
    gbs = inbound / (ms * 1e-3) / 1e9
    return {"kernel": "dp_p2p_kernel<W, sharded optimiser>" if tr.sharded else "dp_p2p_kernel<W, all-reduce>", "floats": count, "ms": ms,
            "nvlink_inbound_bytes": inbound,
            "roofline": {"bound": "nvlink", "achieved": gbs, "peak": 770.0, "unit": "GB/s", "frac": gbs / 770.0,
                         "peak_note": "measured peer-copy bandwidth per direction on this pool (nominal 900)"}}


def measure_cnn(h, rank, world, local_rank, timed, args, rng, gen):
    """CIFAR-shaped CNN, data parallel (global batch 256 split by images over the ranks)."""
    import numpy as np
    import torch

    from tenmo_b200.cnn import CNNTrainer
    from tenmo_b200.parallel import exchange_unique_id, shard_rows, torch_all_gather_bytes, torch_broadcast_bytes

    torch.cuda.nvtx.range_push("cnn")
    gbc = 256
    lo, hi = shard_rows(gbc, rank, world)
    he = lambda shape, fan_in: (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    cp = {"conv1.weight": he((32, 3, 3, 3), 27), "conv1.bias": np.zeros(32, np.float32),
          "conv2.weight": he((64, 32, 3, 3), 288), "conv2.bias": np.zeros(64, np.float32),
          "fc.weight": he((4096, 10), 4096), "fc.bias": np.zeros(10, np.float32)}
    dev = torch.device("cuda", local_rank)
    uid = exchange_unique_id(h.dp_get_unique_id, rank, world, torch_broadcast_bytes(dev)) if args.dp_exchange == "nccl" else None
    def build(exchange, unique_id):
        return CNNTrainer(cp, batch=hi - lo, handle=h, rank=rank, world=world, unique_id=unique_id, device=local_rank,
                          exchange=exchange, all_gather_bytes=torch_all_gather_bytes(dev))

    cnn = build_with_fallback(build, args.dp_exchange, uid, h, rank, world, dev)
    Xc = torch.rand(gbc, 3, 32, 32, generator=gen)[lo:hi].contiguous().pin_memory()
    yc = torch.randint(0, 10, (gbc,), generator=gen)[lo:hi].contiguous().pin_memory()
    cnn.load_batch(Xc, yc)
    for _ in range(3):
        cnn.step()
    check = training_check(cnn, world, dev)
    ms = timed(cnn.step, args.mlp_steps)
    h.check_device_status()
    res = {
        "metric": "cnn_train_samples_per_s", "value": gbc * args.mlp_steps / (ms * 1e-3), "unit": "samples/s",
        "ms_per_step": ms / args.mlp_steps, "scaling": "strong", "global_batch": gbc, "per_rank_batch": hi - lo,
        "steps": args.mlp_steps, "check_after_3_steps": check,
        "config": "(256,3,32,32) U[0,1): conv3x3 3->32 pad1, ReLU, maxpool2, conv3x3 32->64 pad1, ReLU, maxpool2, "
                  "Linear 4096->10, softmax-CE, SGD momentum 0.9; convolutions by the implicit-GEMM kernels (strict fp32, ReLU mask fused into the backward loads)",
    }
    res["exchange"] = cnn.exchange
    if world > 1:
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier()
        cnn.close()
        dist.barrier()
    del cnn
    torch.cuda.empty_cache()
    torch.cuda.nvtx.range_pop()
    return res


def measure_mnist_mlp(h, local_rank, timed, uniform_init, gen):
    """MNIST-shaped MLP on one GPU, the step replayed as a CUDA graph."""
    import numpy as np
    import torch

    from tenmo_b200.trainer import MLPTrainer

    torch.cuda.nvtx.range_push("mnist_mlp")
    dims = [784, 128, 32, 10]
    Ws, bs = uniform_init(dims, lambda i, o: np.sqrt(6.0 / (i + o)))  # Xavier-uniform (net.mojo:87-116)
    tr = MLPTrainer(Ws, bs, batch=64, lr=0.01, momentum=0.9, algo="simt", handle=h, device=local_rank)
    pool = torch.rand(938 * 64, 784, generator=gen).cuda()   # one epoch of synthetic pixels in [0,1)
    labels = torch.randint(0, 10, (938 * 64,), generator=gen).cuda()
    tr.load_batch(pool[:64], labels[:64])
    tr.capture()
    k = [0]

    def epoch_step():
        i = k[0] % 938
        tr.load_batch(pool[i * 64:(i + 1) * 64], labels[i * 64:(i + 1) * 64])
        tr.replay()
        k[0] += 1

    for _ in range(20):
        epoch_step()
    ms = timed(epoch_step, 938)
    res = {
        "metric": "mlp_train_samples_per_s", "value": 938 * 64 / (ms * 1e-3), "unit": "samples/s",
        "us_per_step": ms / 938 * 1e3, "steps": 938, "batch": 64, "final_loss": tr.loss_value(),
        "config": "784-128-32-10 Linear+ReLU, softmax-CE, SGD lr 0.01 momentum 0.9, strict-fp32 GEMMs, one epoch "
                  "(938 steps) of synthetic U[0,1) pixels, step replayed as a CUDA graph; latency-bound",
    }
    h.set_stream(torch.cuda.current_stream(local_rank).cuda_stream)
    h.check_device_status()
    if not getattr(measure_mnist_mlp, "no_cpu", False):
        res["cpu_baseline"] = cpu_mlp_baseline(dims, Ws, bs, pool[:64 * 100].cpu().numpy().reshape(100, 64, 784),
                                               labels[:64 * 100].cpu().numpy().reshape(100, 64), steps=100,
                                               note="MNIST-shaped MLP, 100 steps of batch 64", threads=1)
    torch.cuda.nvtx.range_pop()
    return res


def training_check(tr, world, dev):
    """Loss of the step just run (mean over the ranks) and checksums of the parameters it left, identical inputs at
    every N.  With the NCCL exchange the figures agree with one GPU to ~1e-5; with the peer-memory exchange every
    rank must hold the same bits (max - min of the checksum over the ranks is reported and must be 0)."""
    import torch
    import torch.distributed as dist

    torch.cuda.synchronize()
    loss = tr.loss.detach().double().clone()
    p64 = tr.P.detach().double()
    sums = torch.stack([p64.sum(), p64.abs().sum()])
    spread = 0.0
    if world > 1:
        dist.all_reduce(loss)
        loss /= world
        hi, lo = sums.clone(), sums.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        spread = float((hi - lo).abs().max().item())
    return {"loss": float(loss.item()), "param_sum": float(sums[0].item()), "param_abs_sum": float(sums[1].item()),
            "checksum_spread_over_ranks": spread}


def cpu_mlp_baseline(dims, Ws, bs, X, y, steps, note, threads=None):
    """The oracle's restated Linear/ReLU/cross-entropy/backward/SGD step loop (net.mojo:179-216, optim.mojo:123-158)
    timed on the host's cores for a bounded number of steps; X is (rows, in) for one repeated batch or
    (steps, rows, in) for a sequence of batches."""
    from oracle import ref

    threads = threads or host_cores()
    mlp = ref.MLP(Ws, bs)
    seq = X.ndim == 3
    rows = X.shape[-2]
    mlp.step(X[0] if seq else X, y[0] if seq else y, threads=threads)   # warm up (loads the library)
    t0 = time.perf_counter()
    for i in range(steps):
        mlp.step(X[i] if seq else X, y[i] if seq else y, threads=threads)
    dt = time.perf_counter() - t0
    return {"value": rows * steps / dt, "unit": "samples/s", "cores": threads, "kind": "port",
            "sample": f"{note}: {steps} steps in {dt:.2f} s through the oracle's MLP step ({threads} threads over row tiles)"}


def measure_tf32_yardstick(S=8192, loop=30):
    """A ruler, not part of the path: cuBLAS TF32 GEMMs (torch.matmul with TF32 allowed) at S^3 in this process, CUDA
    events on the current stream -- the best single launch ("burst") and a back-to-back loop of `loop` launches
    ("sustained", the like-for-like figure for a kernel timed inside a long step).  3xTF32 spends three tensor-core
    products per fp32 product, so the roofline of the fp32-accurate GEMM is this figure / 3."""
    import torch

    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a, b = torch.randn(S, S, device="cuda"), torch.randn(S, S, device="cuda")
        c = torch.empty(S, S, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(loop):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / loop
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    flop = 2.0 * S ** 3
    del a, b, c
    torch.cuda.empty_cache()
    return {"burst": flop / (best * 1e-3) / 1e12, "sustained": flop / (sustained_ms * 1e-3) / 1e12, "size": S, "loop": loop,
            "how": "torch.matmul fp32 with TF32 allowed (cuBLAS), CUDA events, same process"}


def measure_simt_fp32(h, timed, S=8192, steps=4):
    """The strict-fp32 arm at the headline size: fwd+bwd through the plain call with the SIMT algorithm, against
    2 x 128 lanes x SMs x the SM clock sampled while it runs (time x clock, not the maximum clock)."""
    import torch

    from tenmo_b200 import ALGO_SIMT_FP32, make_mat

    A, B, dC = (torch.randn(S, S, device="cuda") for _ in range(3))
    C, dA, dB = (torch.empty(S, S, device="cuda") for _ in range(3))
    mA, mB, mdC = (make_mat(t.data_ptr(), (S, S), (S, 1)) for t in (A, B, dC))
    mBt, mAt = make_mat(B.data_ptr(), (S, S), (1, S)), make_mat(A.data_ptr(), (S, S), (1, S))

    def step():
        h.gemm(S, S, S, mA, mB, C.data_ptr(), algo=ALGO_SIMT_FP32)
        h.gemm(S, S, S, mdC, mBt, dA.data_ptr(), algo=ALGO_SIMT_FP32)
        h.gemm(S, S, S, mAt, mdC, dB.data_ptr(), algo=ALGO_SIMT_FP32)

    for _ in range(2):
        step()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    sampler.wait_first()
    t0 = time.time()
    ms = timed(step, steps)
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    kernel = h.gemm_last_kernel()
    info = h.device_info()
    mhz = clocks.get("sm_mhz") or info["sm_clock_khz"] / 1e3
    peak = 2.0 * 128 * info["sm_count"] * mhz * 1e6 / 1e12
    tflops = 6.0 * S ** 3 * steps / (ms * 1e-3) / 1e12
    del A, B, dC, C, dA, dB
    torch.cuda.empty_cache()
    return {"tflops": tflops, "ms_per_step": ms / steps, "kernel": kernel, "size": S,
            "roofline": {"bound": "fp32", "achieved": tflops, "peak": peak, "unit": UNIT, "frac": tflops / peak,
                         "peak_note": f"2 x 128 lanes x {info['sm_count']} SMs x {mhz:.0f} MHz (median SM clock sampled during the run)"},
            "clocks": clocks}


def measure_attention(h, timed, steps=5):
    """Attention-shaped batched products at full size, forward + backward, device-resident, on both kernels:
    S = Q.K^T (K^T a stride view), P.V, and their four backward products, for 384 heads of (512, 64); plus
    (32,512,768)@(1,768,768) with its two backward products.  The (384,512,512) score matrix is 403 MB: its traffic
    bounds the 3xTF32 numbers, so the GB/s it moves at is reported beside the TFLOP/s."""
    import torch

    from tenmo_b200 import ALGO_SIMT_FP32, ALGO_TC_3XTF32, make_mat

    BH, S, D = 384, 512, 64
    f32 = dict(dtype=torch.float32, device="cuda")
    q, k, v, dctx = (torch.randn(BH, S, D, **f32) * 0.125 for _ in range(4))
    sc, dsc = torch.empty(BH, S, S, **f32), torch.randn(BH, S, S, **f32)
    ctx, dq, dk, dv = (torch.empty(BH, S, D, **f32) for _ in range(4))
    dp = torch.empty(BH, S, S, **f32)
    b3 = lambda t, r, c, rs, cs: make_mat(t.data_ptr(), (BH, r, c), (t.stride(0), rs, cs))
    out = {}
    for name, algo in (("3xtf32", ALGO_TC_3XTF32), ("simt", ALGO_SIMT_FP32)):
        def step():
            h.gemm(S, S, D, b3(q, S, D, D, 1), b3(k, D, S, 1, D), sc.data_ptr(), algo=algo)        # scores = Q . K^T
            h.gemm(S, D, S, b3(sc, S, S, S, 1), b3(v, S, D, D, 1), ctx.data_ptr(), algo=algo)      # ctx = P . V
            h.gemm(S, D, S, b3(sc, S, S, 1, S), b3(dctx, S, D, D, 1), dv.data_ptr(), algo=algo)    # dV = P^T . dctx
            h.gemm(S, S, D, b3(dctx, S, D, D, 1), b3(v, D, S, 1, D), dp.data_ptr(), algo=algo)     # dP = dctx . V^T
            h.gemm(S, D, S, b3(dsc, S, S, S, 1), b3(k, S, D, D, 1), dq.data_ptr(), algo=algo)      # dQ = dS . K
            h.gemm(S, D, S, b3(dsc, S, S, 1, S), b3(q, S, D, D, 1), dk.data_ptr(), algo=algo)      # dK = dS^T . Q

        for _ in range(2):
            step()
        ms = timed(step, steps) / steps
        flop = 6 * 2.0 * BH * S * S * D
        # score-sized matrices moved per step: scores written, read by P.V and by dV, dP written, dS read twice
        score_bytes = 6 * 4.0 * BH * S * S
        out[name] = {"ms_per_step": ms, "tflops": flop / (ms * 1e-3) / 1e12, "score_matrix_gbs": score_bytes / (ms * 1e-3) / 1e9}
    del q, k, v, dctx, sc, dsc, ctx, dq, dk, dv, dp
    torch.cuda.empty_cache()
    Bb, M, K, N = 32, 512, 768, 768
    a, w, dc = torch.randn(Bb, M, K, **f32) * 0.05, torch.randn(1, K, N, **f32) * 0.05, torch.randn(Bb, M, N, **f32)
    c, da, dw_full, dw = torch.empty(Bb, M, N, **f32), torch.empty(Bb, M, K, **f32), torch.empty(Bb, K, N, **f32), torch.empty(K, N, **f32)
    for name, algo in (("3xtf32", ALGO_TC_3XTF32), ("simt", ALGO_SIMT_FP32)):
        def step():
            h.gemm(M, N, K, make_mat(a.data_ptr(), (Bb, M, K), (M * K, K, 1)), make_mat(w.data_ptr(), (1, K, N), (K * N, N, 1)),
                   c.data_ptr(), algo=algo)
            h.gemm(M, K, N, make_mat(dc.data_ptr(), (Bb, M, N), (M * N, N, 1)), make_mat(w.data_ptr(), (1, N, K), (K * N, 1, N)),
                   da.data_ptr(), algo=algo)
            h.gemm(K, N, M, make_mat(a.data_ptr(), (Bb, K, M), (M * K, 1, K)), make_mat(dc.data_ptr(), (Bb, M, N), (M * N, N, 1)),
                   dw_full.data_ptr(), algo=algo)
            h.colsum(dw_full.data_ptr(), Bb, K * N, K * N, dw.data_ptr())   # sum over the broadcast batch

        for _ in range(2):
            step()
        ms = timed(step, steps) / steps
        out[name]["broadcast_batched_ms_per_step"] = ms
        out[name]["broadcast_batched_tflops"] = 6.0 * Bb * M * K * N / (ms * 1e-3) / 1e12
    out["config"] = ("384 x (512,64).(64,512)-view then .(512,64) and the four backward products; "
                     "(32,512,768)@(1,768,768) with dA and dB summed over the batch; N(0, 1/sqrt(64)) / N(0, 0.05^2) inputs")
    h.check_device_status()
    return out


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from tenmo_b200 import ALGO_SIMT_FP32, ALGO_TC_3XTF32, TenmoCuda, make_mat

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    h = TenmoCuda(local_rank).require()  # fails loudly if the CUDA library is missing: there is no fallback
    stream = torch.cuda.current_stream()
    h.set_stream(stream.cuda_stream)
    algo = ALGO_SIMT_FP32 if args.algo == "simt" else ALGO_TC_3XTF32

    S = args.size
    M = N = K = S
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host_in = [torch.randn(S, S, generator=gen, dtype=torch.float32).pin_memory() for _ in range(3)]  # A, B, dC
    host_out = [torch.empty(S, S, dtype=torch.float32).pin_memory() for _ in range(3)]               # C, dA, dB
    A, B, dC = (t.cuda(non_blocking=True) for t in host_in)
    C, dA, dB = (torch.empty(S, S, device="cuda") for _ in range(3))
    torch.cuda.synchronize()

    def mats(a, b, dc):
        mA = make_mat(a.data_ptr(), (M, K), (K, 1))
        mB = make_mat(b.data_ptr(), (K, N), (N, 1))
        mBt = make_mat(b.data_ptr(), (N, K), (1, N))    # B^T as a stride view
        mAt = make_mat(a.data_ptr(), (K, M), (1, K))    # A^T as a stride view
        mdC = make_mat(dc.data_ptr(), (M, N), (N, 1))
        return mA, mB, mBt, mAt, mdC

    mA, mB, mBt, mAt, mdC = mats(A, B, dC)

    # 3xTF32: each input is split into its lo plane once per step (the transposed view of a matrix shares the plane of
    # its storage) and the three GEMMs are handed the planes; the plain tenmo_gemm_f32 call would split both operands
    # of every GEMM again.  Strict fp32 has no planes.
    use_planes = algo == ALGO_TC_3XTF32

    def new_planes():
        return tuple(torch.empty(S * S, device="cuda") for _ in range(3)) if use_planes else None

    def run_step(m, outs, planes):
        m_a, m_b, m_bt, m_at, m_dc = m
        c, da, db = outs
        if not use_planes:
            h.gemm(M, N, K, m_a, m_b, c.data_ptr(), algo=algo)       # C  = A . B
            h.gemm(M, K, N, m_dc, m_bt, da.data_ptr(), algo=algo)    # dA = dC . B^T
            h.gemm(K, N, M, m_at, m_dc, db.data_ptr(), algo=algo)    # dB = A^T . dC
            return
        a_lo, b_lo, dc_lo = (t.data_ptr() for t in planes)
        h.split_lo(m_a, M, K, a_lo, S * S)
        h.split_lo(m_b, K, N, b_lo, S * S)
        h.gemm_ex(M, N, K, m_a, m_b, c.data_ptr(), algo=algo, a_lo=a_lo, b_lo=b_lo)
        h.split_lo(m_dc, M, N, dc_lo, S * S)
        h.gemm_ex(M, K, N, m_dc, m_bt, da.data_ptr(), algo=algo, a_lo=dc_lo, b_lo=b_lo)
        h.gemm_ex(K, N, M, m_at, m_dc, db.data_ptr(), algo=algo, a_lo=a_lo, b_lo=dc_lo)

    planes0 = new_planes()

    def step_device():
        run_step((mA, mB, mBt, mAt, mdC), (C, dA, dB), planes0)

    # End to end: every step copies A, B, dC from pinned host memory and reads C, dA, dB back.  The copies run on their
    # own streams and two sets of device buffers alternate, so that the uploads of step i+1 and the read-back of step
    # i-1 overlap the GEMMs of step i (PCIe is full duplex); events carry the dependencies operand by operand.
    s_h2d, s_d2h = torch.cuda.Stream(), torch.cuda.Stream()
    sets = [dict(inp=(A, B, dC), out=(C, dA, dB))]
    sets.append(dict(inp=tuple(torch.empty_like(t) for t in (A, B, dC)), out=tuple(torch.empty_like(t) for t in (C, dA, dB))))
    for st in sets:
        st["mats"] = mats(*st["inp"])
        st["planes"] = planes0 if st is sets[0] else new_planes()
        st["ev_ab"], st["ev_dc"], st["ev_c"], st["ev_da"], st["ev_db"], st["ev_read"] = (torch.cuda.Event() for _ in range(6))
        st["used"] = False
    e2e_count = [0]

    def step_e2e():
        st = sets[e2e_count[0] % 2]
        e2e_count[0] += 1
        a, b, dc = st["inp"]
        c, da, db = st["out"]
        m_a, m_b, m_bt, m_at, m_dc = st["mats"]
        with torch.cuda.stream(s_h2d):
            if st["used"]:
                s_h2d.wait_event(st["ev_db"])          # the GEMMs that last read this set's inputs are done
            a.copy_(host_in[0], non_blocking=True)
            b.copy_(host_in[1], non_blocking=True)
            st["ev_ab"].record(s_h2d)
            dc.copy_(host_in[2], non_blocking=True)
            st["ev_dc"].record(s_h2d)
        if st["used"]:
            stream.wait_event(st["ev_read"])           # this set's previous results have been read back
        stream.wait_event(st["ev_ab"])
        if use_planes:
            a_lo, b_lo, dc_lo = (t.data_ptr() for t in st["planes"])
            h.split_lo(m_a, M, K, a_lo, S * S)
            h.split_lo(m_b, K, N, b_lo, S * S)
            h.gemm_ex(M, N, K, m_a, m_b, c.data_ptr(), algo=algo, a_lo=a_lo, b_lo=b_lo)
        else:
            h.gemm(M, N, K, m_a, m_b, c.data_ptr(), algo=algo)
        st["ev_c"].record(stream)
        stream.wait_event(st["ev_dc"])
        if use_planes:
            h.split_lo(m_dc, M, N, dc_lo, S * S)
            h.gemm_ex(M, K, N, m_dc, m_bt, da.data_ptr(), algo=algo, a_lo=dc_lo, b_lo=b_lo)
        else:
            h.gemm(M, K, N, m_dc, m_bt, da.data_ptr(), algo=algo)
        st["ev_da"].record(stream)
        if use_planes:
            h.gemm_ex(K, N, M, m_at, m_dc, db.data_ptr(), algo=algo, a_lo=a_lo, b_lo=dc_lo)
        else:
            h.gemm(K, N, M, m_at, m_dc, db.data_ptr(), algo=algo)
        st["ev_db"].record(stream)
        with torch.cuda.stream(s_d2h):
            s_d2h.wait_event(st["ev_c"])
            host_out[0].copy_(c, non_blocking=True)
            s_d2h.wait_event(st["ev_da"])
            host_out[1].copy_(da, non_blocking=True)
            s_d2h.wait_event(st["ev_db"])
            host_out[2].copy_(db, non_blocking=True)
            st["ev_read"].record(s_d2h)
        st["used"] = True

    def e2e_join():
        """Make the timing stream wait for every read-back issued so far."""
        for st in sets:
            if st["used"]:
                stream.wait_event(st["ev_read"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        if fn is step_e2e:
            e2e_join()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        barrier()
        return float(ms.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.wait_first()
    h.launch_count(reset=True)
    h.profile_begin()
    t_begin = time.time()
    ms_dev = timed(step_device, args.steps)
    t_end = time.time()
    launches = h.launch_count(reset=True)
    n_kernel, kernel_ms = h.profile_end()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    h.check_device_status()
    last_kernel = h.gemm_last_kernel()  # which GEMM kernel the steps above launched

    # release the GEMM buffers before the MLP legs
    del A, B, dC, C, dA, dB, host_in, host_out, sets, planes0
    torch.cuda.empty_cache()
    sweep = None if (args.no_sweep or world > 1) else measure_other_sizes(h, algo, timed)
    extras = {}
    if world == 1 and not args.no_extras:
        yard = measure_tf32_yardstick(S)
        extras["simt_fp32"] = measure_simt_fp32(h, timed, S)
        extras["attention"] = measure_attention(h, timed)
        hbm = {}
        run_kernel_rooflines(args, h=h, collect=hbm)
        extras["hbm_kernels"] = hbm
        h.set_stream(stream.cuda_stream)
    else:
        yard = None
    mlp = None if args.no_mlp else measure_mlps(h, rank, world, local_rank, timed, args)

    flop_step = 6.0 * M * N * K
    value = flop_step * world * args.steps / (ms_dev * 1e-3) / 1e12
    e2e_value = flop_step * world * args.steps / (ms_e2e * 1e-3) / 1e12
    peaks = load_peaks()
    if args.algo == "simt":
        info = h.device_info()
        peak = 2.0 * 128 * info["sm_count"] * info["sm_clock_khz"] * 1e3 / 1e12
        peak_note = "strict-FP32 SIMT peak = 2 x 128 lanes x SMs x max SM clock"
        kernel = last_kernel or "gemm_simt_kernel"
    else:
        peak_bf16 = peaks["bf16_sustained"] / 2.0 / 3.0
        if yard:
            peak = yard["sustained"] / 3.0
            peak_note = (f"TF32 GEMM measured in this run (cuBLAS, {yard['loop']} back-to-back {yard['size']}^3 launches): "
                         f"{yard['sustained']:.1f} TFLOP/s / 3 (three tensor-core products per fp32 product); best single launch "
                         f"{yard['burst']:.1f} / 3 = {yard['burst'] / 3.0:.1f}; derived from the {peaks['source']} bf16 peak: "
                         f"{peaks['bf16_sustained']:.1f} / 2 / 3 = {peak_bf16:.1f} sustained, {peaks['bf16_burst'] / 6.0:.1f} burst")
        else:
            peak = peak_bf16
            peak_note = (f"{peaks['source']} bf16 sustained {peaks['bf16_sustained']:.1f} TFLOP/s / 2 (TF32 rate) / 3 "
                         f"(three products per fp32 product); burst-based figure {peaks['bf16_burst'] / 6.0:.1f}")
        kernel = last_kernel or "gemm_tc_kernel"
    achieved = (2.0 * M * N * K) / ((kernel_ms / max(n_kernel, 1)) * 1e-3) / 1e12 if n_kernel else None

    out = None
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": gemm_workload_text(S), "size": S, "algo": "3xtf32-tcgen05" if algo == 1 else "simt-fp32",
                       "parallelism": f"replicas x{world}", "l2": "inputs (3 x %.0f MB) exceed the 126 MB L2" % (S * S * 4 / 1e6)},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": 3 * S * S * 4, "d2h_bytes_per_step": 3 * S * S * 4,
                    "note": "pinned host buffers; uploads, GEMMs and read-backs on three streams over two sets of device "
                            "buffers, so neighbouring steps overlap; timed until the last read-back has landed"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor" if algo == 1 else "fp32", "kernel": kernel, "achieved": achieved, "peak": peak,
                         "unit": UNIT, "frac": (achieved / peak) if achieved else None,
                         "traffic": NCU_TRAFFIC_BYTES.get((kernel, S)), "traffic_unit": "bytes per launch (ncu, dram read+write)",
                         "launches_timed": n_kernel, "avg_launch_ms": kernel_ms / max(n_kernel, 1), "peak_note": peak_note},
        }
        if yard and algo == 1:
            out["roofline"]["tf32_measured"] = yard["sustained"]
            out["roofline"]["tf32_measured_burst"] = yard["burst"]
            out["roofline"]["frac_of_bf16_derived_sustained"] = achieved / peak_bf16 if achieved else None
            out["roofline"]["frac_of_bf16_derived_burst"] = achieved / (peaks["bf16_burst"] / 6.0) if achieved else None
        out["e2e"]["pcie_note"] = ("805 MB each way per step and rank: the end-to-end figure is bound by the host link, and at N > 1 "
                                   "all ranks share the host's memory and PCIe paths")
        out.update(extras)
        if sweep:
            out["other_sizes"] = sweep
        if mlp:
            out.update(mlp)
        if world == 1 and not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline(args.cpu_budget)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------
# HBM-bound kernels of the path against the bandwidth roofline
# ---------------------------------------------------------------------------------------------------
def run_kernel_rooflines(args, h=None, collect=None):
    """One JSON line per kernel (or one entry of ``collect``): algorithmic bytes per launch / CUDA-event time, against
    the measured copy bandwidth.  Shapes are the wide-MLP ones (per-rank batch 8192).  Every kernel cycles through
    enough distinct buffers that the working set exceeds the 126 MB L2."""
    import torch

    from tenmo_b200 import TenmoCuda, make_mat

    if h is None:
        torch.cuda.set_device(0)
        h = TenmoCuda(0).require()
    stream = torch.cuda.current_stream()
    h.set_stream(stream.cuda_stream)
    peaks = load_peaks()
    f32 = dict(dtype=torch.float32, device="cuda")

    def report(name, alg_bytes, fn, iters=40, note=""):
        for i in range(5):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(iters):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        gbs = alg_bytes / (ms * 1e-3) / 1e9
        entry = {"kernel": name, "avg_launch_ms": ms, "roofline": {
            "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
            "traffic": NCU_TRAFFIC_BYTES.get((name, 8192 * 4096)), "peak_note": f"{peaks['source']} copy bandwidth"},
            "algorithmic_bytes": alg_bytes,
            "note": note}
        if collect is not None:
            collect[name] = {"gbs": gbs, "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal_8tbs": gbs / 8000.0,
                             "avg_launch_ms": ms, "algorithmic_bytes": alg_bytes, "note": note}
        else:
            print(json.dumps(entry), flush=True)

    M, N, C = 8192, 4096, 1000
    R = 4  # rotating buffers: 4 x 134 MB
    xs = [torch.randn(M, N, **f32) for _ in range(R)]
    out = torch.empty(N, **f32)
    report("colsum_split_kernel", 4.0 * M * N + 4.0 * N,
           lambda i: h.colsum(xs[i % R].data_ptr(), M, N, N, out.data_ptr()), note=f"bias gradient of a ({M},{N}) activation gradient")
    ys = [torch.empty(M, N, **f32) for _ in range(2)]
    report("ew_kernel<relu_bwd>", 12.0 * M * N,
           lambda i: h.relu_bwd(xs[i % R].data_ptr(), xs[(i + 1) % R].data_ptr(), ys[i % 2].data_ptr(), M * N),
           note="dx = g * mask")
    report("add_bias_kernel", 8.0 * M * N + 4.0 * N,
           lambda i: h.add_bias(xs[i % R].data_ptr(), out.data_ptr(), ys[i % 2].data_ptr(), M, N), note="un-fused bias add")
    del ys
    # SGD over the wide MLP's 54.4 M parameters (218 MB each of p, g, v)
    n = 54440936
    p, g, v = (torch.randn(n, **f32) * 0.01 for _ in range(3))
    report("sgd_kernel", 20.0 * n, lambda i: h.sgd_step([p.data_ptr()], [g.data_ptr()], [v.data_ptr()], [n], 0.01, 0.9, 0.0, 1.0),
           note="momentum 0.9, one flat tensor of 54.4 M parameters")
    del p, g, v, xs
    # cross-entropy at (8192, 1000): 32 MB per matrix, so rotate 8 logits / softmax pairs
    R = 8
    logits = [torch.randn(M, C, **f32) for _ in range(R)]
    sm = [torch.empty(M, C, **f32) for _ in range(R)]
    labels = torch.randint(0, C, (M,), device="cuda")
    loss, valid = torch.zeros(1, **f32), torch.zeros(1, dtype=torch.int32, device="cuda")
    report("ce_fwd_stream_kernel", 8.0 * M * C + 8.0 * M,
           lambda i: h.ce_fwd(logits[i % R].data_ptr(), C, labels.data_ptr(), True, M, C, -100, 0.0, 0, sm[i % R].data_ptr(),
                              loss.data_ptr(), valid.data_ptr()), note="softmax kept for backward, loss finished on the device")
    report("ce_bwd_kernel", 8.0 * M * C + 8.0 * M,
           lambda i: h.ce_bwd(sm[i % R].data_ptr(), labels.data_ptr(), True, M, C, -100, 0.0, 0, 0, valid.data_ptr(),
                              logits[i % R].data_ptr()))
    del logits, sm
    # matrix @ vector and vector @ matrix on a (65536, 4096) matrix (1 GB: larger than the L2 by itself)
    Mr, Kc = 65536, 4096
    A = torch.randn(Mr, Kc, **f32)
    xv, yv = torch.randn(Kc, **f32), torch.empty(Mr, **f32)
    xr, yc = torch.randn(Mr, **f32), torch.empty(Kc, **f32)
    mA = make_mat(A.data_ptr(), (Mr, Kc), (Kc, 1))
    report("gemv_kernel", 4.0 * Mr * Kc + 4.0 * (Mr + Kc), lambda i: h.gemv(Mr, Kc, mA, xv.data_ptr(), 1, yv.data_ptr()),
           iters=20, note="y = A . x, A (65536, 4096) row-major")
    report("vecmat_kernel", 4.0 * Mr * Kc + 4.0 * (Mr + Kc), lambda i: h.vecmat(Mr, Kc, xr.data_ptr(), 1, mA, yc.data_ptr()),
           iters=20, note="y = x . A, A (65536, 4096) row-major")
    del A
    torch.cuda.empty_cache()
    h.check_device_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--algo", choices=["tc", "simt"], default="tc")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--ref-size", type=int, default=0, help="force the CPU sample size of --impl reference (0 = --size if it fits --ref-budget)")
    ap.add_argument("--ref-budget", type=float, default=150.0, help="seconds the whole --impl reference run may take")
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-mlp", action="store_true", help="skip the MLP training legs")
    ap.add_argument("--no-sweep", action="store_true", help="skip the smaller / skinny GEMM sizes of the same configuration")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the TF32 yardstick, the strict-fp32 arm, the attention shapes and the HBM-bound kernels")
    ap.add_argument("--mlp-steps", type=int, default=20)
    ap.add_argument("--dp-exchange", choices=["auto", "nccl", "p2p", "p2p_allreduce"], default="auto",
                    help="gradient exchange of the training legs at N > 1: NCCL all-reduce or the library's peer-memory kernel; "
                         "auto = peer-memory from 8 ranks up (measured: 17 %% faster at 8 ranks, 6 %% slower at 4, 5 %% slower at 2)")
    ap.add_argument("--dp-overlap", action="store_true", help="force the per-layer exchange onto a side stream beside the backward GEMMs")
    ap.add_argument("--dp-no-overlap", action="store_true",
                    help="run the gradient exchange after the backward pass on the compute stream (for measuring what the overlap hides)")
    ap.add_argument("--legs", default="wide_mlp,cnn,mnist_mlp", help="which training legs to run after the GEMM arm")
    ap.add_argument("--kernels", action="store_true",
                    help="time the bandwidth-bound kernels of the path against the HBM roofline (one JSON line each)")
    args = ap.parse_args()
    if args.dp_exchange == "auto":
        args.dp_exchange = "p2p" if int(os.environ.get("WORLD_SIZE", "1")) >= 8 else "nccl"
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.kernels:
        run_kernel_rooflines(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
