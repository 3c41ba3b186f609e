#!/usr/bin/env python3
"""Benchmark of the Converse2D forward hot path and of the networks built on it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--dtype fp32|bf16]
                    [--models all|none|name,...]

Headline workload (N=1 and per GPU at N>1): one Converse2D upsampling layer, C=64, k=5, scale 2,
circular padding 2, input 16x64x64x64 -> output 16x64x128x128, seeded N(0,1) input,
softmax-normalised taps, zero bias.  A step is one forward over that batch.  Rank 0 prints ONE
JSON line.

`value` times the C-ABI call with inputs resident in HBM: CUDA events on the launch stream, K steps
captured in a CUDA graph (launch latency is not the number), the block of K steps repeated until the
timed region is several hundred milliseconds long; `ms_per_step` is the median over the blocks (min /
max / mean in `detail`).  `e2e` times the module API from pinned host buffers with both copies
inside the timed region, `e2e.copy_ceiling` the same copies without the kernel.  The same line
carries the layer with the other element type (`bf16`), the single-image layer (`cfg1`), and
`models`: images/s of Converse-DnCNN, -SRResNet and -USRNet (scale 1 and 4) at the batch sizes of
the benchmark configurations, the batch sharded over the ranks.

`--impl reference` times the reference's own CPU path on the host cores: its C++ operator
(oracle/_ref, compiled from the reference's source) for the layer, and the restated reference
networks (oracle/ref_networks.py) for `models`.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=16, C=64, H=64, W=64, k=5, s=2, p=2, mode="circular", eps=1e-5)
WORKLOAD = "converse2d_fwd cfg2: B16 C64 64x64 -> 128x128, k5 s2 p2 circular"
CFG1 = dict(B=1, C=64, H=128, W=128, k=5, s=1, p=2, mode="circular", eps=1e-5)
WORKLOAD1 = "converse2d_fwd cfg1: B1 C64 128x128, k5 s1 p2 circular"
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(cfg, esize):
    n_in = cfg["B"] * cfg["C"] * cfg["H"] * cfg["W"]
    return n_in * esize + n_in * cfg["s"] ** 2 * esize


def out_pixels(cfg):
    return cfg["B"] * cfg["C"] * cfg["H"] * cfg["W"] * cfg["s"] ** 2


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def seeded_case(cfg, seed=0):
    import numpy as np
    from oracle import converse2d_oracle as orc
    rng = np.random.default_rng(seed)
    w, b = orc.init_weight(cfg["C"], cfg["k"], rng)
    x = rng.standard_normal((cfg["B"], cfg["C"], cfg["H"], cfg["W"])).astype(np.float32)
    return x, w, b


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ whole networks
MODEL_CFG = {
    # name: global batch, input shape per image, scale factor fed to the network (USRNet only), fp32
    # algorithmic GB per global batch with the fusion-forced accounting (11*C*H*W*e per ConverseBlock:
    # LN+1x1+GELU reads C writes 2C, Converse2D reads 2C writes 2C, the rest reads 2C+C writes C)
    "dncnn": dict(batch=8, shape=(1, 256, 256), sf=None, gbytes=29.8,
                  desc="Converse-DnCNN, B8 x 1 x 256 x 256 (config 3)"),
    "srresnet": dict(batch=16, shape=(3, 128, 128), sf=None, gbytes=30.2,
                     desc="Converse-SRResNet x4, B16 x 3 x 128 x 128 -> 512 x 512 (config 4)"),
    "usrnet_sf1": dict(batch=32, shape=(3, 512, 512), sf=1, gbytes=853.0,
                       desc="Converse-USRNet sf1, B32 x 3 x 512 x 512 (config 5)"),
    "usrnet_sf4": dict(batch=32, shape=(3, 128, 128), sf=4, gbytes=853.0 - 1.6,
                       desc="Converse-USRNet sf4, B32 x 3 x 128 x 128 -> 512 x 512 (config 5)"),
    "conversenet": dict(batch=8, shape=(3, 256, 256), sf=None, gbytes=8 * 35 * 11 * 64 * 256 * 256 * 4 / 1e9,
                        desc="ConverseNet (blind variant), B8 x 3 x 256 x 256"),
}


def anisotropic_gaussian_kernel(rng, size=25):
    """Seeded anisotropic Gaussian blur kernel: sigma_x, sigma_y ~ U[0.6, 5], rotation ~ U[0, pi),
    normalised to sum 1 (the recipe of the reference's `utils/utils_sisr.py:35-66,172-213`)."""
    import numpy as np
    sx, sy, th = rng.uniform(0.6, 5.0), rng.uniform(0.6, 5.0), rng.uniform(0.0, np.pi)
    c, s_ = np.cos(th), np.sin(th)
    rot = np.array([[c, -s_], [s_, c]])
    inv = np.linalg.inv(rot @ np.diag([sx * sx, sy * sy]) @ rot.T)
    r = np.arange(size) - size // 2
    yy, xx = np.meshgrid(r, r, indexing="ij")
    u = np.stack([xx, yy], axis=-1).astype(np.float64)
    k = np.exp(-0.5 * np.einsum("...i,ij,...j->...", u, inv, u))
    return k / k.sum()


def synthetic_batch(name, n, seed):
    """Seeded stand-ins for the missing image sets, with the shapes and value distributions the
    configs name.  Returns (x float32 (n,c,h,w), extra) where extra = () or (k (n,1,7,7), sf).

    dncnn: N(0,1) field, Gaussian-filtered sigma 3 px, min-max to [0,1], + N(0, (25/255)^2).
    srresnet / conversenet: U[0,1] smoothed with a 3x3 box filter.
    usrnet: smooth random image blurred (wrap-around) with a 25x25 anisotropic Gaussian kernel,
      decimated by sf, + N(0, sigma^2) with sigma ~ U[0, 7.65]/255 per image; the network is fed the
      central 7x7 crop of the kernel renormalised to sum 1, because the reference's KernelNet accepts
      7x7 kernels only (`models/converse_usrnet.py:126-131`)."""
    import numpy as np
    from scipy.ndimage import gaussian_filter, uniform_filter
    rng = np.random.default_rng(seed)
    mc = MODEL_CFG[name]
    c, h, w = mc["shape"]
    if name == "dncnn":
        f = gaussian_filter(rng.standard_normal((n, c, h, w)), sigma=(0, 0, 3, 3))
        f = (f - f.min()) / (f.max() - f.min())
        return (f + rng.standard_normal(f.shape) * 25.0 / 255.0).astype(np.float32), ()
    if name in ("srresnet", "conversenet"):
        return uniform_filter(rng.uniform(size=(n, c, h, w)), size=(1, 1, 3, 3)).astype(np.float32), ()
    sf = mc["sf"]
    H, W = h * sf, w * sf
    xs, ks = [], []
    for _ in range(n):
        img = gaussian_filter(rng.standard_normal((c, H, W)), sigma=(0, 4, 4))
        img = (img - img.min()) / (img.max() - img.min())
        k25 = anisotropic_gaussian_kernel(rng)
        pad = np.zeros((H, W))
        pad[:25, :25] = k25
        pad = np.roll(pad, (-12, -12), axis=(0, 1))
        blurred = np.fft.irfft2(np.fft.rfft2(img) * np.fft.rfft2(pad)[None], s=(H, W))
        low = blurred[:, ::sf, ::sf]
        low = low + rng.standard_normal(low.shape) * rng.uniform(0.0, 7.65 / 255.0)
        k7 = k25[9:16, 9:16]
        xs.append(low)
        ks.append(k7 / k7.sum())
    return np.stack(xs).astype(np.float32), (np.stack(ks)[:, None].astype(np.float32), sf)


BENCH_MODELS = ["dncnn", "srresnet", "usrnet_sf1", "usrnet_sf4"]


# ------------------------------------------------------------------ CPU side: the reference's own path
def load_reference_op():
    """Register the reference's C++ operator (oracle/_ref, compiled from the reference's source) in
    this process.  False when the file is absent: callers then use the torch.fft restatement."""
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "converse2d_ref.so")
    if not os.path.exists(so):
        return False
    if not (hasattr(torch.ops, "converse2d") and hasattr(torch.ops.converse2d, "forward")):
        torch.ops.load_library(so)
    return True


def reference_layer_fn(cfg, device="cpu"):
    """One Converse2D layer the way the reference runs it: the module-side glue of
    `models/util_converse.py:144-145,166,189-190` around its C++ op (or, without oracle/_ref, the
    torch.fft restatement in oracle/ref_networks.py).  Returns (callable on a torch tensor, kind)."""
    import torch
    import torch.nn.functional as F
    from oracle import ref_networks as rn
    _, w, b = seeded_case(cfg)
    wt, bt = torch.from_numpy(w).to(device), torch.from_numpy(b).to(device)
    p, s, mode, eps = cfg["p"], cfg["s"], cfg["mode"], cfg["eps"]
    have_op = load_reference_op()

    def run(xt):
        y = F.pad(xt, [p, p, p, p], mode=mode) if p > 0 else xt
        x0 = y if s == 1 else F.interpolate(y, scale_factor=s, mode="nearest")
        if have_op:
            out = torch.ops.converse2d.forward(y, x0, wt, bt, s, eps)
        else:
            out = rn.solve(y, x0, wt, torch.sigmoid(bt - 9.0) + eps, s)
        return out[..., p * s:-p * s, p * s:-p * s] if p > 0 else out

    return run, ("reference" if have_op else "port")


def time_cpu_layer(cfg, budget_s, steps=5, warmup=1):
    """The layer on the host cores, on a bounded sample: the leading batch entries that fit the
    budget.  Returns (Mpix/s, info)."""
    import torch
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    fn, kind = reference_layer_fn(cfg)
    x = torch.from_numpy(seeded_case(cfg)[0])
    B = x.shape[0]
    with torch.no_grad():
        t0 = time.perf_counter()
        fn(x[:1])
        t1 = time.perf_counter() - t0
        bs = int(max(1, min(B, budget_s / max(1, steps + warmup) / max(t1, 1e-6))))
        xs = x[:bs]
        for _ in range(warmup):
            fn(xs)
        ts = []
        for _ in range(steps):
            t0 = time.perf_counter()
            fn(xs)
            ts.append(time.perf_counter() - t0)
    t = statistics.mean(ts)
    pix = bs * cfg["C"] * cfg["H"] * cfg["W"] * cfg["s"] ** 2
    return pix / t / 1e6, {"kind": kind, "cores": threads, "ms_per_step": t * 1e3,
                           "sample": "first %d of %d batch entries, %d timed steps, mean" % (bs, B, steps)}


def seed_alphas(net, seed=5):
    """The alpha-variant blocks and the data step of ConverseUSRNet start at zero
    (`models/util_converse.py:303-304`): draw them so that a random-init network uses its blocks."""
    import torch
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in net.named_parameters():
            if n.endswith("alpha1") or n.endswith("alpha2"):
                p.copy_(0.1 * torch.randn(p.shape, generator=g))
            elif n.endswith("d.alpha"):
                p.copy_(9.0 + torch.randn(p.shape, generator=g))


def network_name(workload):
    return "usrnet" if workload.startswith("usrnet") else workload


def oracle_network(workload, device="cpu"):
    """The restated reference network (oracle/ref_networks.py) with seeded random-init weights."""
    import torch
    from oracle import ref_networks as rn
    torch.manual_seed(0)
    net = rn.NETWORKS[network_name(workload)]()
    seed_alphas(net)
    rn.use_reference_op(load_reference_op())
    return net.to(device).eval()


def time_cpu_model(workload, reps=1):
    """images/s of the reference network on the host cores, batch 1.  USRNet is sampled: one of its
    five identical unrolled iterations (data step + seven blocks) is timed and scaled by five."""
    import torch
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    net = oracle_network(workload)
    x, extra = synthetic_batch(workload, 1, 100)
    xt = torch.from_numpy(x)
    with torch.no_grad():
        if network_name(workload) == "usrnet":
            kt, sf = torch.from_numpy(extra[0]), extra[1]
            kk = net.kernelnet(kt)
            feat = net.conv1(xt)
            if sf != 1:   # the timed iteration runs at the output resolution, as four of the five do
                feat = torch.nn.functional.interpolate(feat, scale_factor=sf, mode="nearest")
            kc = net.convs[1](kk).view(1, 64, 7, 7)
            t0 = time.perf_counter()
            for _ in range(reps):
                net.p(net.d(feat, kc, 1))
            t = (time.perf_counter() - t0) / reps * 5.0
            sample = "batch 1: one of 5 unrolled iterations (data step + 7 blocks) timed %dx, scaled by 5" % reps
        else:
            t0 = time.perf_counter()
            for _ in range(reps):
                net(xt)
            t = (time.perf_counter() - t0) / reps
            sample = "batch 1, %d forward(s), mean" % reps
    from oracle import ref_networks as rn
    return {"value": 1.0 / t, "unit": "images/s", "cores": threads, "kind": "port",
            "sample": sample + ("; Converse2D layers through the reference's C++ op" if rn._use_ref_op else "")}


def base_line(args, impl=None):
    line = {"metric": "converse2d_fwd_throughput", "value": None, "unit": "Mpix/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "pixels": "B*C*sH*sW output plane-pixels"}}
    if impl:
        line = dict({"impl": impl}, **line)
    return line


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    val, info = time_cpu_layer(CFG, budget_s=90.0, steps=max(1, args.steps), warmup=max(1, min(args.warmup, 3)))
    line = base_line(args, "reference")
    line.update({
        "value": val, "ms_per_step": info["ms_per_step"],
        "cpu_baseline": {"value": val, "unit": "Mpix/s", "cores": info["cores"], "kind": info["kind"],
                         "sample": info["sample"]},
        "e2e": {"value": val, "unit": "Mpix/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    if args.models != "none":
        models = {}
        for name in selected_models(args):
            try:
                cb = time_cpu_model(name)
                models[name] = {"images_per_s": cb["value"], "workload": MODEL_CFG[name]["desc"],
                                "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "images/s",
                                                            "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
            except Exception as e:
                models[name] = {"unavailable": "%s: %s" % (type(e).__name__, e)}
        line["models"] = models
    print(json.dumps(line))


def selected_models(args):
    if args.models in ("all", ""):
        return list(BENCH_MODELS)
    if args.models == "none":
        return []
    names = [n for n in args.models.split(",") if n]
    for n in names:
        if n not in MODEL_CFG:
            raise SystemExit("unknown model workload %r (known: %s)" % (n, ", ".join(MODEL_CFG)))
    return names


# ------------------------------------------------------------------ our arm (GPU)
class Ranks:
    """Rank bookkeeping: one process per GPU, NCCL only for barriers and the max-over-ranks of times."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (no CPU path exists for the product)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.affinity = bind_near_gpu(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ms(self, ms):
        from conversenet_b200.sharding import max_over_ranks
        return max_over_ranks(ms, device=self.dev) if self.world > 1 else float(ms)

    def close(self):
        import torch.distributed as dist
        if self.world > 1:
            dist.destroy_process_group()


def bind_near_gpu(local):
    """Pin this process to the CPUs of its GPU's NUMA node (pinned-buffer copies are driven from
    there).  Best effort: returns a description, or None when the topology cannot be read."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        dom = torch.cuda.get_device_properties(local).pci_domain_id
        dev_id = torch.cuda.get_device_properties(local).pci_device_id
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/local_cpulist" % (dom, bus, dev_id)
        with open(path) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
        return {"local_cpulist": text, "bound": len(cpus) if cpus else len(allowed)}
    except Exception:
        return None


def layer_module(cfg, dev):
    import torch
    from conversenet_b200 import Converse2D
    _, w_np, b_np = seeded_case(cfg)
    mod = Converse2D(cfg["C"], cfg["C"], cfg["k"], scale=cfg["s"], padding=cfg["p"],
                     padding_mode=cfg["mode"], eps=cfg["eps"]).to(dev).eval()
    with torch.no_grad():
        mod.weight.copy_(torch.from_numpy(w_np))
        mod.bias.copy_(torch.from_numpy(b_np))
    return mod


def time_layer(R, cfg, dtype, K, W, target_ms, use_graph=True, check=False):
    """Device-timed forward of one layer through the C ABI, inputs resident in HBM.

    K steps (rotating buffer sets, together larger than L2) form one block, captured in a CUDA graph;
    the block is replayed back to back until about `target_ms` have passed, an event between blocks.
    Returns per-step milliseconds (median / min / max over the blocks, max over ranks of the median)."""
    import torch
    from conversenet_b200 import functional as CF
    dev = R.dev
    tdtype = torch.float32 if dtype == "fp32" else torch.bfloat16
    esize = 4 if dtype == "fp32" else 2
    x_np = seeded_case(cfg)[0]
    mod = layer_module(cfg, dev)
    step_bytes = algorithmic_bytes(cfg, esize)
    nbuf = max(2, -(-2 * L2_BYTES // step_bytes) + 1)
    x_host = torch.from_numpy(x_np).to(tdtype)
    xs = [x_host.to(dev) if i == 0 else (x_host.to(dev) * (1.0 + 0.001 * i)).to(tdtype) for i in range(nbuf)]
    outs = [torch.empty((cfg["B"], cfg["C"], cfg["H"] * cfg["s"], cfg["W"] * cfg["s"]), dtype=tdtype, device=dev)
            for _ in range(nbuf)]
    h, w = cfg["H"] + 2 * cfg["p"], cfg["W"] + 2 * cfg["p"]
    table, wf = mod._table_for(h, w, dev)

    def step(i):
        CF.converse2d_forward(xs[i % nbuf], table, wf, cfg["k"], cfg["s"], cfg["p"], cfg["mode"], out=outs[i % nbuf])

    for i in range(max(W, 3)):
        step(i)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    g = None
    if use_graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    for i in range(K):
                        step(i)
        except Exception as e:  # eager launches, still timed on the device
            g = None
            sys.stderr.write("graph capture failed (%s); timing eager launches\n" % e)
    torch.cuda.synchronize()

    def block():
        if g is not None:
            g.replay()
        else:
            for i in range(K):
                step(i)

    # size the run from a short probe
    with torch.cuda.stream(stream):
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        block()
        block()
        p1.record(stream)
    stream.synchronize()
    probe = max(p0.elapsed_time(p1) / 2.0, 1e-3)
    nblocks = int(min(20000, max(5, -(-target_ms // probe))))
    sampler = ClockSampler(R.local)
    R.barrier()
    sampler.start()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(nblocks + 1)]
    with torch.cuda.stream(stream):
        evs[0].record(stream)
        for b in range(nblocks):
            block()
            evs[b + 1].record(stream)
    stream.synchronize()
    R.barrier()
    clocks = sampler.stop()
    per_block = [evs[b].elapsed_time(evs[b + 1]) for b in range(nblocks)]
    med = statistics.median(per_block) / K
    res = {"ms_per_step": R.max_ms(med), "ms_per_step_rank": med, "ms_min": min(per_block) / K,
           "ms_max": max(per_block) / K, "ms_mean": evs[0].elapsed_time(evs[nblocks]) / (nblocks * K),
           "blocks": nblocks, "launches": nblocks * K, "graph": g is not None, "nbuf": nbuf,
           "step_bytes": step_bytes, "clocks": clocks, "timed_ms": evs[0].elapsed_time(evs[nblocks])}
    if check:
        import numpy as np
        from oracle import converse2d_oracle as orc
        _, w_np, b_np = seeded_case(cfg)
        want = orc.converse2d_forward(x_np[:1], w_np, b_np, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"],
                                      dtype=np.float64)
        res["rel_l2_vs_oracle"] = orc.rel_l2(outs[0][:1].float().cpu().numpy(), want)
    res["_mod"], res["_x_host"], res["_out_shape"] = mod, x_host, tuple(outs[0].shape)
    return res


def e2e_layer(R, mod, x_host, out_shape, Ke, with_kernel=True):
    """The module API from pinned host memory: every step copies its input in and its result out;
    the copies of neighbouring steps overlap on two copy streams, the kernel runs between.
    `with_kernel=False` moves the same bytes on the same streams without the kernel (the ceiling
    the copies alone set)."""
    import torch
    dev = R.dev
    tdtype = x_host.dtype
    xh = x_host.pin_memory()
    ohs = [torch.empty(out_shape, dtype=tdtype).pin_memory() for _ in range(2)]
    xds = [torch.empty(x_host.shape, dtype=tdtype, device=dev) for _ in range(2)]
    yds = [torch.empty(out_shape, dtype=tdtype, device=dev) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    done = [None, None]

    def one(i):
        b = i & 1
        if done[b] is not None:
            s_in.wait_event(done[b])
        with torch.cuda.stream(s_in):
            xds[b].copy_(xh, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        main.wait_event(ev_in)
        if with_kernel:
            with torch.no_grad():
                y = mod(xds[b])
        else:
            y = yds[b]
        done[b] = torch.cuda.Event()
        done[b].record(main)
        s_out.wait_event(done[b])
        with torch.cuda.stream(s_out):
            ohs[b].copy_(y, non_blocking=True)
        y.record_stream(s_out)

    for i in range(4):
        one(i)
    main.wait_stream(s_out)
    R.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    s_in.wait_event(e0)
    for i in range(Ke):
        one(i)
    main.wait_stream(s_out)
    main.wait_stream(s_in)
    e1.record()
    torch.cuda.synchronize()
    if with_kernel:
        with torch.no_grad():
            if not torch.equal(ohs[(Ke - 1) & 1], mod(xds[0]).cpu()):
                raise RuntimeError("end-to-end result differs from the resident run")
    R.barrier()
    ms = R.max_ms(e0.elapsed_time(e1)) / Ke
    return ms, x_host.numel() * x_host.element_size(), ohs[0].numel() * ohs[0].element_size()


def product_network(workload, dev, tdtype):
    import torch
    from conversenet_b200 import models
    ctor = {"dncnn": models.ConverseDnCNN, "srresnet": models.ConverseMSRResNet, "usrnet": models.ConverseUSRNet,
            "conversenet": models.ConverseNet}[network_name(workload)]
    torch.manual_seed(0)
    net = ctor()
    seed_alphas(net)
    net = net.to(dev).eval()
    if tdtype != torch.float32:
        if hasattr(net, "activation_dtype"):
            net.activation_dtype = tdtype    # fp32 parameters, bf16 tensors between the body's kernels
        else:
            net = net.to(tdtype)
    return net


def time_model(R, workload, dtype="fp32", target_ms=1500.0, args_no_graph=False):
    """images/s of a whole network: the global batch of the configuration cut into contiguous slices
    over the ranks (`conversenet_b200.sharding.shard_batch`: slices differ by at most one image; with
    fewer images than ranks the last ranks idle), weights replicated, no collective."""
    import torch
    from conversenet_b200.sharding import shard_batch
    mc = MODEL_CFG[workload]
    dev = R.dev
    tdtype = torch.float32 if dtype == "fp32" else torch.bfloat16
    start, count = shard_batch(mc["batch"], R.rank, R.world)
    net = product_network(workload, dev, tdtype)
    xh, kd, sf, out = None, None, None, None
    if count > 0:
        x, extra = synthetic_batch(workload, count, 100 + R.rank)
        xh = torch.from_numpy(x).to(tdtype).pin_memory()
        if extra:
            kd, sf = torch.from_numpy(extra[0]).to(dev), extra[1]

    def eager(xd):
        return net(xd, kd, sf) if kd is not None else net(xd)

    fwd, launch = eager, "eager"
    with torch.no_grad():
        xd = xh.to(dev) if count else None
        if count and not args_no_graph:
            # one CUDA-graph launch per forward instead of hundreds of kernel launches
            try:
                from conversenet_b200.graphs import GraphedForward
                gf = GraphedForward(net, *([xd, kd, sf] if kd is not None else [xd]))
                fwd = (lambda t: gf(t, kd, sf)) if kd is not None else (lambda t: gf(t))
                launch = "cuda graph replay"
            except Exception as e:
                sys.stderr.write("graph capture of %s failed (%s); timing eager launches\n" % (workload, e))
                torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(3):   # warm-up: tables, workspaces, allocator
            if i == 2:
                t0.record()
            if count:
                out = fwd(xd)
        t1.record()
        torch.cuda.synchronize()
        probe = R.max_ms(max(t0.elapsed_time(t1), 1e-3))
        Km = int(min(50, max(3, -(-target_ms // probe))))
        sampler = ClockSampler(R.local)
        R.barrier()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(Km):
            if count:
                out = fwd(xd)
        e1.record()
        torch.cuda.synchronize()
        R.barrier()
        clocks = sampler.stop()
        ms_step = R.max_ms(e0.elapsed_time(e1)) / Km
        # end to end: pinned host input in, host output back, every step
        Ke = max(2, min(Km, 5))
        oh = torch.empty(out.shape, dtype=out.dtype).pin_memory() if count else None
        xin = torch.empty_like(xd) if count else None
        R.barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(Ke):
            if count:
                xin.copy_(xh, non_blocking=True)
                oh.copy_(fwd(xin), non_blocking=True)
        f1.record()
        torch.cuda.synchronize()
        R.barrier()
        ms_e2e = R.max_ms(f0.elapsed_time(f1)) / Ke
    peak, peak_kind = measured_peak_gbs()
    esize = 4 if dtype == "fp32" else 2
    gb_rank = mc["gbytes"] * (count / mc["batch"]) * esize / 4.0   # this rank's algorithmic bytes per step
    busiest = mc["gbytes"] * (shard_batch(mc["batch"], 0, R.world)[1] / mc["batch"]) * esize / 4.0
    achieved = busiest / (ms_step * 1e-3)
    del gb_rank
    res = {
        "workload": mc["desc"], "images_per_s": mc["batch"] / (ms_step * 1e-3), "ms_per_step": ms_step,
        "global_batch": mc["batch"], "per_rank_batch": [shard_batch(mc["batch"], r, R.world)[1] for r in range(R.world)],
        "steps": Km, "warmup": 3, "scaling": "strong", "dtype": "f32" if dtype == "fp32" else "bf16", "launch": launch,
        "e2e": {"value": mc["batch"] / (ms_e2e * 1e-3), "unit": "images/s", "steps": Ke,
                "h2d_bytes_per_step": (xh.numel() * xh.element_size()) if count else 0,
                "d2h_bytes_per_step": (oh.numel() * oh.element_size()) if count else 0},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_kind,
                     "note": "fusion-forced algorithmic bytes of the busiest rank / step time"},
        "clocks": clocks,
    }
    del net, out, fwd
    torch.cuda.empty_cache()
    return res


def gpu_library_baseline(R, cfg, K=20):
    """The reference's operator on CUDA tensors of the same GPU (its C++ op = ATen + cuFFT, TF32 off):
    the library path the hand-written kernels replace.  Rank 0 at N=1."""
    import torch
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        fn, kind = reference_layer_fn(cfg, R.dev)
        x = torch.from_numpy(seeded_case(cfg)[0]).to(R.dev)
        with torch.no_grad():
            for _ in range(3):
                fn(x)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                fn(x)
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / K
        return {"value": out_pixels(cfg) / (ms * 1e-3) / 1e6, "unit": "Mpix/s", "ms_per_step": ms, "kind": kind,
                "what": "reference Converse2D op on CUDA tensors (ATen + cuFFT), same layer, same GPU, TF32 off",
                "steps": K}
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32


def train_step_layer(R, cfg, K=20):
    """Forward + backward (dL/dx, dL/dweight, dL/dbias) of the configuration's layer through the module, ms per
    step, beside the same step with the operator written entirely in `torch.fft` (cuFFT + ATen, TF32 off) on the
    same GPU.  The reference trains through the latter.  Rank 0 at N=1; a side figure, not the headline."""
    import torch
    from conversenet_b200 import Converse2D
    from conversenet_b200.autograd import spectral_forward
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        m = Converse2D(cfg["C"], cfg["C"], cfg["k"], scale=cfg["s"], padding=cfg["p"], padding_mode=cfg["mode"],
                       eps=cfg["eps"]).to(R.dev)
        x = torch.from_numpy(seeded_case(cfg)[0]).to(R.dev).requires_grad_(True)
        g = torch.randn(cfg["B"], cfg["C"], cfg["H"] * cfg["s"], cfg["W"] * cfg["s"], device=R.dev) * 1e-4

        def ours():
            torch.autograd.grad(m(x), (x, m.weight, m.bias), g)

        def library():
            y = spectral_forward(x, m.weight, m.bias, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
            torch.autograd.grad(y, (x, m.weight, m.bias), g)

        out = {}
        for name, fn in (("ms_per_step", ours), ("torch_fft_ms_per_step", library)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                fn()
            e1.record()
            torch.cuda.synchronize()
            out[name] = e0.elapsed_time(e1) / K
        out["what"] = ("forward + dL/dx + dL/dweight + dL/dbias of the headline layer through the module "
                       "(native kernels; the chain rule on the (C,h,w) multiplier in PyTorch) against the operator "
                       "written in torch.fft under autograd; both bound by host launches")
        out["steps"] = K
        return out
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32


def gpu_library_model(R, workload, batch):
    """The restated reference network on CUDA tensors (torch.fft -> cuFFT, ATen, cuDNN 1x1; TF32 off)."""
    import torch
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        net = oracle_network(workload, R.dev)
        x, extra = synthetic_batch(workload, batch, 100)
        args = [torch.from_numpy(x).to(R.dev)]
        if extra:
            args += [torch.from_numpy(extra[0]).to(R.dev), extra[1]]
        with torch.no_grad():
            net(*args)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(2):
                net(*args)
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 2
        del net
        torch.cuda.empty_cache()
        return {"images_per_s": batch / (ms * 1e-3), "batch": batch, "ms_per_step": ms,
                "what": "restated reference network on CUDA tensors (cuFFT + ATen + cuDNN), TF32 off"}
    except Exception as e:
        torch.cuda.empty_cache()
        return {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32


def run_ours(args):
    import torch
    from conversenet_b200 import _cabi
    R = Ranks()
    _cabi.load()
    torch.backends.cudnn.allow_tf32 = False       # the networks' few non-fused 1x1 convolutions stay fp32
    torch.backends.cuda.matmul.allow_tf32 = False
    K, W = max(1, args.steps), args.warmup
    peak, peak_kind = measured_peak_gbs()
    first, second = ("fp32", "bf16") if args.dtype == "fp32" else ("bf16", "fp32")

    t = time_layer(R, CFG, first, K, W, args.target_ms, use_graph=not args.no_graph, check=True)
    ms_step = t["ms_per_step"]
    value = R.world * out_pixels(CFG) / (ms_step * 1e-3) / 1e6
    achieved = t["step_bytes"] / (t["ms_per_step_rank"] * 1e-3) / 1e9
    line = base_line(args)
    line.update({
        "value": value, "n_gpus": R.world, "ms_per_step": ms_step,
        "dtype": "f32" if first == "fp32" else "bf16-io/f32",
        "detail": {"mpix_per_s_reference_definition": value / CFG["C"],
                   "l2": "%d rotating buffer sets (%.0f MB) > L2" % (t["nbuf"], t["nbuf"] * t["step_bytes"] / 1e6),
                   "launch": "cuda graph replay" if t["graph"] else "eager", "io_dtype": first,
                   "sharding": "each rank runs the full batch on its own planes; no collective",
                   "timed_region_ms": t["timed_ms"], "blocks_of_K_steps": t["blocks"],
                   "ms_per_step_min": t["ms_min"], "ms_per_step_max": t["ms_max"], "ms_per_step_mean": t["ms_mean"],
                   "ms_per_step_is": "median over blocks, max over ranks",
                   "rel_l2_vs_oracle": t["rel_l2_vs_oracle"], "cpu_affinity": R.affinity},
        "clocks": t["clocks"], "gpu_launches": t["launches"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": read_traffic(), "peak_source": peak_kind,
                     "algorithmic_bytes_per_launch": t["step_bytes"]},
    })
    if args.kernel_only:
        if R.rank == 0:
            print(json.dumps(line))
        R.close()
        return
    Ke = max(3, min(K, 20))
    ms_e2e, bi, bo = e2e_layer(R, t["_mod"], t["_x_host"], t["_out_shape"], Ke)
    ms_copy, _, _ = e2e_layer(R, t["_mod"], t["_x_host"], t["_out_shape"], Ke, with_kernel=False)
    line["e2e"] = {"value": R.world * out_pixels(CFG) / (ms_e2e * 1e-3) / 1e6, "unit": "Mpix/s",
                   "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo, "steps": Ke, "ms_per_step": ms_e2e,
                   "pipeline": "H2D of step i+1 and D2H of step i overlap on copy streams",
                   "copy_ceiling": {"value": R.world * out_pixels(CFG) / (ms_copy * 1e-3) / 1e6, "unit": "Mpix/s",
                                    "ms_per_step": ms_copy,
                                    "what": "the same copies on the same streams with no kernel between them"}}
    del t
    torch.cuda.empty_cache()

    # the other element type of the same layer, and the small single-image layer (config 1)
    t2 = time_layer(R, CFG, second, K, W, args.target_ms / 4, use_graph=not args.no_graph)
    b2 = t2["step_bytes"]
    line["bf16" if second == "bf16" else "fp32"] = {
        "value": R.world * out_pixels(CFG) / (t2["ms_per_step"] * 1e-3) / 1e6, "unit": "Mpix/s",
        "ms_per_step": t2["ms_per_step"], "dtype": "bf16-io/f32" if second == "bf16" else "f32",
        "roofline": {"achieved": b2 / (t2["ms_per_step_rank"] * 1e-3) / 1e9, "peak": peak,
                     "frac": b2 / (t2["ms_per_step_rank"] * 1e-3) / 1e9 / peak, "algorithmic_bytes_per_launch": b2}}
    del t2
    t1 = time_layer(R, CFG1, "fp32", K, W, args.target_ms / 8, use_graph=not args.no_graph)
    b1 = t1["step_bytes"]
    line["cfg1"] = {"workload": WORKLOAD1, "value": R.world * out_pixels(CFG1) / (t1["ms_per_step"] * 1e-3) / 1e6,
                    "unit": "Mpix/s", "ms_per_step": t1["ms_per_step"],
                    "roofline": {"achieved": b1 / (t1["ms_per_step_rank"] * 1e-3) / 1e9, "peak": peak,
                                 "frac": b1 / (t1["ms_per_step_rank"] * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes_per_launch": b1}}
    del t1
    torch.cuda.empty_cache()

    models = {}
    for name in selected_models(args):
        try:
            models[name] = time_model(R, name, "fp32", args_no_graph=args.no_graph)
        except Exception as e:   # one network failing must not lose the line
            models[name] = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}
            torch.cuda.empty_cache()
    if "dncnn" in models and args.models != "none" and "unavailable" not in models["dncnn"]:
        try:
            models["dncnn_bf16"] = time_model(R, "dncnn", "bf16", target_ms=500.0, args_no_graph=args.no_graph)
        except Exception as e:
            models["dncnn_bf16"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}
    if models:
        line["models"] = models

    if R.rank == 0 and R.world == 1 and not args.no_baselines:
        try:
            line["gpu_library_baseline"] = gpu_library_baseline(R, CFG)
            for name, batch in (("dncnn", 8), ("srresnet", 16), ("usrnet_sf1", 4)):
                if name in models:
                    models[name]["gpu_library_baseline"] = gpu_library_model(R, name, batch)
        except Exception as e:
            line["gpu_library_baseline"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
        try:
            line["train_step"] = train_step_layer(R, CFG)
        except Exception as e:
            line["train_step"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
        try:
            v, info = time_cpu_layer(CFG, budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": "Mpix/s", "cores": info["cores"], "kind": info["kind"],
                                    "sample": info["sample"]}
            for name in models:
                if name in MODEL_CFG and name in ("dncnn", "srresnet", "usrnet_sf1"):
                    models[name]["cpu_baseline"] = time_cpu_model(name)
        except Exception as e:
            line.setdefault("cpu_baseline", {"value": None, "unit": "Mpix/s", "cores": 0, "kind": "port",
                                             "sample": "failed: %s" % e})
    if R.rank == 0:
        print(json.dumps(line))
    R.close()


def profile_model(args):
    """Two forwards of one network workload (the first builds tables and workspaces), nothing timed:
    the command a profiler wraps."""
    import torch
    R = Ranks()
    name = args.profile_model
    mc = MODEL_CFG[name]
    tdtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    net = product_network(name, R.dev, tdtype)
    batch = args.profile_batch or (mc["batch"] if not name.startswith("usrnet") else 4)
    x, extra = synthetic_batch(name, batch, 100)
    xs = [torch.from_numpy(x).to(R.dev).to(tdtype)]
    if extra:
        xs += [torch.from_numpy(extra[0]).to(R.dev), extra[1]]
    with torch.no_grad():
        for _ in range(2):
            y = net(*xs)
    torch.cuda.synchronize()
    print(json.dumps({"profile_model": name, "out_shape": list(y.shape), "finite": bool(torch.isfinite(y).all())}))
    R.close()


def read_traffic():
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get("converse2d_fwd_cfg2_dram_bytes_per_launch")
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--models", default="all",
                    help="'all', 'none', or a comma list of %s: the network workloads reported in the "
                         "line's \"models\" object" % ", ".join(MODEL_CFG))
    ap.add_argument("--target-ms", type=float, default=600.0,
                    help="length of the timed region of the headline layer (blocks of --steps steps are repeated)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-baselines", action="store_true", help="skip the CPU and library baselines")
    ap.add_argument("--profile-model", default="",
                    help="run only two forwards of one network workload at its benchmark batch (profiler runs)")
    ap.add_argument("--profile-batch", type=int, default=0,
                    help="batch of the --profile-model forwards (default: the workload's per-GPU batch)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the headline layer's device-timed part (for profiler runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.profile_model:
        profile_model(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
