#!/usr/bin/env python
"""Benchmark of the delta-rule hot path on B200.

Workload (N=1): chunk_gdn2 training forward+backward at the headline shape
B=1, L=2048, Hk=12, Hv=24, K=V=128, bf16 q/k/v, fp32 gates, precision='bf16',
chunk 128, qk_l2norm, documents split at L/2, all six gradients -- plus the decode
step on 256 sequences x 32 value heads x (128x128) bf16 state.  Inputs are seeded
synthetic tensors with the reference benchmark's distributions.

One JSON line is printed by rank 0:
  value        tokens/s of fwd+bwd with inputs resident in HBM (all GPUs together),
  e2e          the same through the public Python operator with HOST buffers (pinned H2D of
               the inputs and D2H of out + all gradients of every timed step inside the timed
               region; batches are double-buffered, so one step's copies overlap its neighbours'
               compute; the unpipelined time per step is reported beside it),
  roofline     the dominant kernel of the step against the measured peak,
  decode       state-stream GB/s of the decode step with its own roofline,
  cpu_baseline the CPU oracle (a port of the reference's chunked path) on the host cores.

`--only sp` runs a different workload and prints its own line: KDA-style fwd+bwd on one packed
sequence of 131072 tokens, split over the ranks (strong scaling; the state chain crosses the ranks
by NCCL point-to-point).

`--impl reference` times the CPU oracle instead (the reference itself needs an array
library that is not installed on the box; the oracle restates its chunked algorithm).
With N>1 GPUs every rank runs the same per-GPU workload on its own data (batch
sharding: no collective on the data path), so scaling is weak.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "deltanet-tpu_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

CFG = dict(B=1, L=2048, Hk=12, Hv=24, K=128, V=128, chunk=128)
DEC = dict(B=256, Hk=16, Hv=32, K=128, V=128)


# ------------------------------------------------------------------------------------------ peaks
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------------------------------ flops
def alg_flops(c):
    """Algorithmic dense-matmul FLOPs per chunk-head of each kernel of this build.

    The terms are those of the reference kernels (prepass fwd: A and M on the lower blocks,
    the triangular inverse at C^3/3, W, U; state fwd: 3 state products + M V_new; state bwd:
    7 state products + 2 CxC products; prepass bwd) regrouped by the kernel that performs
    them here: the reverse chain keeps 3 state products + M^T dO, the chunk-parallel
    backward takes the other 4 state products + dO V_new^T and the whole prepass adjoint.
    """
    C, K, Vw = c["chunk"], c["K"], (c["Hv"] // c["Hk"]) * c["V"]
    ns = C // 32
    f = (ns + 1) / (2 * ns)
    pre_fwd = 2 * f * 2 * C * C * K + C ** 3 / 3 + 2 * C * C * K + 2 * C * C * Vw
    st_fwd = 3 * 2 * C * K * Vw + 2 * C * C * Vw
    chain_bwd = 3 * 2 * C * K * Vw + 2 * C * C * Vw
    pre_bwd_ref = 2 * 2 * C * C * K + 2 * 2 * C * C * Vw + 2 * 2 * C ** 3 + 4 * ((ns - 1) / (2 * ns)) * 2 * C * C * K
    par_bwd = 4 * 2 * C * K * Vw + 2 * C * C * Vw + pre_bwd_ref
    return dict(prepass_fwd=pre_fwd, state_fwd=st_fwd, state_bwd=chain_bwd, prepass_bwd=par_bwd)


def alg_bytes(c):
    """Algorithmic HBM bytes per (batch, exec head, chunk) item and kernel: every array the kernel must
    read or write, once (bf16 q/k/v/out/dO and residual tiles, fp32 gates, T, states, dV, dH)."""
    C, K, Vw = c["chunk"], c["K"], (c["Hv"] // c["Hk"]) * c["V"]
    qk, gb, vv, ww = 2 * C * K * 2, 2 * C * K * 4, C * Vw * 2, C * Vw * 4
    tiles = 3 * C * K * 2 + C * C * 2 + C * Vw * 2              # W, qe, ke, M, U
    pre_fwd = qk + gb + vv + ww + tiles + C * C * 4 + K * 4
    st_fwd = tiles + C * Vw * 2 + K * Vw * 4                     # + out, chunk-entry state
    chain_bwd = 3 * C * K * 2 + C * C * 2 + C * Vw * 2 + C * Vw * 4 + K * Vw * 4    # tiles, dO -> dV, dH
    par_bwd = (C * K * 2 + C * Vw * 2 + K * Vw * 4 + C * C * 4 + C * Vw * 2 + C * Vw * 4 + K * Vw * 4
               + qk + gb + vv + ww + qk + gb + vv + ww)          # W,U,S,T,dO,dV,dH, inputs, six gradients
    return dict(prepass_fwd=pre_fwd, state_fwd=st_fwd, state_bwd=chain_bwd, prepass_bwd=par_bwd)


# dram__bytes_read.sum + dram__bytes_write.sum of a kernel's launches in one step of the headline workload
# (both chunk ranges together), from the ncu capture summarised in profiles/chunk_step_kernels_headline.md
NCU_DRAM_BYTES = {"prepass_bwd": 301.1e6, "prepass_fwd": 82.1e6, "state_fwd": 40.5e6, "state_bwd": 66.2e6}


# ------------------------------------------------------------------------------------------ inputs
def make_training_inputs(seed, c, device=None, pin=False):
    gen = torch.Generator().manual_seed(seed)
    B, L, Hk, Hv, K, V = c["B"], c["L"], c["Hk"], c["Hv"], c["K"], c["V"]
    rn = lambda *s: torch.randn(*s, generator=gen)
    t = dict(
        q=rn(B, L, Hk, K).to(torch.bfloat16), k=rn(B, L, Hk, K).to(torch.bfloat16),
        v=rn(B, L, Hv, V).to(torch.bfloat16),
        b=torch.sigmoid(rn(B, L, Hk, K) * 0.39), w=torch.sigmoid(rn(B, L, Hv, V) * 0.39),
        g=-torch.exp(rn(B, L, Hk, K) * 0.39 - 1.0),
        do=rn(B, L, Hv, V).to(torch.bfloat16),
        seg=(torch.arange(L) >= L // 2).to(torch.int32)[None].expand(B, L).contiguous(),
    )
    if pin:
        t = {k_: v_.pin_memory() for k_, v_ in t.items()}
    if device is not None:
        t = {k_: v_.to(device) for k_, v_ in t.items()}
    return t


class DeviceJob:
    """fwd+bwd through the C ABI on pre-allocated device buffers (nothing allocated per step)."""

    def __init__(self, c, dev, seed):
        from deltanet_b200 import _lib as L
        self.L, self.lib = L, L.lib()
        self.t = make_training_inputs(seed, c, device=dev)
        t = self.t
        self.shape = L.Shape(B=c["B"], L=c["L"], Hk=c["Hk"], Hv=c["Hv"], K=c["K"], V=c["V"], chunk=c["chunk"],
                             g_heads=c["Hk"], g_cols=c["K"], b_heads=c["Hk"], b_cols=c["K"],
                             w_heads=c["Hv"], w_cols=c["V"], qkv_dtype=L.DN_BF16, gate_dtype=L.DN_F32,
                             precision=L.DN_PREC_BF16, flags=L.DN_QK_L2NORM, scale=c["K"] ** -0.5)
        self.out = torch.empty_like(t["v"])
        self.grads = {n: torch.empty_like(t[n]) for n in "qkvgbw"}
        self.res_block = torch.empty(self.lib.dn_residual_bytes(self.shape), dtype=torch.uint8, device=dev)
        self.res = L.Residuals()
        L.check(self.lib.dn_residual_carve(self.shape, self.res_block.data_ptr(), self.res), "carve")
        n = max(self.lib.dn_scratch_bytes(self.shape, 0, 0), self.lib.dn_scratch_bytes(self.shape, 1, 0))
        self.scratch = torch.empty(n, dtype=torch.uint8, device=dev)
        ex = L.Exec()
        self.lib.dn_exec_view(self.shape, ex)
        self.ex = ex
        items = c["B"] * ex.H * ex.NC
        self.dV = torch.empty(items * ex.chunk * ex.Vw, dtype=torch.float32, device=dev)
        self.dH = torch.empty(items * c["K"] * ex.Vw, dtype=torch.float32, device=dev)
        self.stream = torch.cuda.current_stream().cuda_stream
        self.bytes = sum(x.numel() * x.element_size() for x in (self.res_block, self.scratch, self.out)) + \
            sum(x.numel() * x.element_size() for x in t.values()) + \
            sum(x.numel() * x.element_size() for x in self.grads.values())

    def _p(self, n):
        return self.t[n].data_ptr()

    def fwd(self):
        L, s, sc = self.L, self.shape, self.scratch
        L.check(self.lib.dn_chunk_fwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                      self._p("w"), self._p("seg"), None, self.out.data_ptr(), None, self.res,
                                      sc.data_ptr(), sc.numel(), self.stream), "dn_chunk_fwd")

    def bwd(self):
        L, s, sc, gr = self.L, self.shape, self.scratch, self.grads
        L.check(self.lib.dn_chunk_bwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                      self._p("w"), self._p("seg"), None, self.res, self._p("do"), None,
                                      gr["q"].data_ptr(), gr["k"].data_ptr(), gr["v"].data_ptr(),
                                      gr["g"].data_ptr(), gr["b"].data_ptr(), gr["w"].data_ptr(), None,
                                      sc.data_ptr(), sc.numel(), self.stream), "dn_chunk_bwd")

    def step(self):
        self.fwd()
        self.bwd()

    # single phases, for the per-kernel timing
    def phase(self, name):
        L, s, sc = self.L, self.shape, self.scratch
        if name == "prepass_fwd":
            L.check(self.lib.dn_prepass_fwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                            self._p("w"), self._p("seg"), self.res, sc.data_ptr(), sc.numel(),
                                            self.stream), name)
        elif name == "state_fwd":
            L.check(self.lib.dn_state_fwd(s, self.res, self._p("seg"), None, self.out.data_ptr(), None, self.stream), name)
        elif name == "state_bwd":
            L.check(self.lib.dn_state_bwd(s, self.res, self._p("seg"), self._p("do"), None, self.dV.data_ptr(),
                                          self.dH.data_ptr(), None, self.stream), name)
        elif name == "prepass_bwd":
            gr = self.grads
            L.check(self.lib.dn_prepass_bwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                            self._p("w"), self._p("seg"), self.res, self._p("do"),
                                            self.dV.data_ptr(), self.dH.data_ptr(), gr["q"].data_ptr(),
                                            gr["k"].data_ptr(), gr["v"].data_ptr(), gr["g"].data_ptr(),
                                            gr["b"].data_ptr(), gr["w"].data_ptr(), sc.data_ptr(), sc.numel(),
                                            self.stream), name)


class DecodeJob:
    def __init__(self, d, dev, seed, heads=None):
        from deltanet_b200 import _lib as L
        self.L, self.lib = L, L.lib()
        Hv = heads or d["Hv"]
        Hk = max(1, Hv * d["Hk"] // d["Hv"])
        B, K, V = d["B"], d["K"], d["V"]
        gen = torch.Generator().manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=gen)
        self.q = rn(B, Hk, K).to(torch.bfloat16).to(dev)
        self.k = rn(B, Hk, K).to(torch.bfloat16).to(dev)
        self.v = rn(B, Hv, V).to(torch.bfloat16).to(dev)
        self.b = torch.sigmoid(rn(B, Hk, K) * 0.39).to(dev)
        self.w = torch.sigmoid(rn(B, Hv, V) * 0.39).to(dev)
        self.g = (-torch.exp(rn(B, Hk, K) * 0.39 - 1.0)).to(dev)
        self.state = [(torch.randn(B, Hv, K, V, device=dev) * 0.1).to(torch.bfloat16) for _ in range(2)]
        self.o = torch.empty(B, Hv, V, dtype=torch.bfloat16, device=dev)
        self.shape = L.DecodeShape(B=B, Hk=Hk, Hv=Hv, K=K, V=V, g_heads=Hk, g_cols=K, b_heads=Hk, b_cols=K,
                                   w_heads=Hv, w_cols=V, qkv_dtype=L.DN_BF16, gate_dtype=L.DN_F32,
                                   state_in_dtype=L.DN_BF16, state_out_dtype=L.DN_BF16, flags=L.DN_QK_L2NORM,
                                   scale=K ** -0.5, stability_tau=1000.0)
        self.state_bytes = 2 * B * Hv * K * V * 2
        self.vec_bytes = sum(x.numel() * x.element_size() for x in (self.q, self.k, self.v, self.b, self.w, self.g, self.o))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.i = 0

    def step(self):
        a, b_ = self.state[self.i & 1], self.state[(self.i + 1) & 1]
        self.i += 1
        self.L.check(self.lib.dn_decode_step(self.shape, self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                                             self.g.data_ptr(), self.b.data_ptr(), self.w.data_ptr(), a.data_ptr(),
                                             None, self.o.data_ptr(), b_.data_ptr(), self.stream), "dn_decode_step")


# ------------------------------------------------------------------------------------------ helpers
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.3)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()

    def summary(self):
        sm = sorted(int(float(r[1])) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [int(float(r[2])) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for nm, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def time_steps(fn, steps, warmup, dist=None):
    """W warm-ups, then K steps between CUDA events on the current stream; max over ranks (ms)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


# ------------------------------------------------------------------------------------------ CPU oracle leg
def cpu_oracle_step(c, heads_frac, seed=11):
    """One fwd+bwd of the oracle's chunked path on a head-subset of the workload; returns seconds."""
    from oracle import delta_oracle as O
    Hk = max(1, int(c["Hk"] * heads_frac))
    Hv = Hk * (c["Hv"] // c["Hk"])
    cc = dict(c, Hk=Hk, Hv=Hv)
    t = make_training_inputs(seed, cc)
    ins = [t[n].clone().requires_grad_() for n in "qkvgbw"]
    t0 = time.perf_counter()
    o = O.chunk_gdn2(*ins, segment_ids=t["seg"], chunk_size=c["chunk"], precision="bf16", qk_l2norm=True)
    torch.autograd.grad((o.float() * t["do"].float()).sum(), ins)
    return time.perf_counter() - t0, Hv / c["Hv"]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    frac = 1.0 / 6.0                       # 2 key heads / 4 value heads of the 12 / 24
    times, budget, t_start = [], 150.0, time.perf_counter()
    for i in range(args.warmup + args.steps):
        dt, f = cpu_oracle_step(CFG, frac)
        if i >= args.warmup:
            times.append(dt)
        if time.perf_counter() - t_start > budget and times:
            break
    sec = sum(times) / len(times)
    tok = CFG["B"] * CFG["L"] * f / sec
    sample = (f"oracle port of the reference's chunked path (gdn2.py:772-1173), torch CPU, {cores} threads; each step = "
              f"fwd+bwd on {int(24 * f)} of 24 value heads at L=2048 (token count scaled by the head fraction); "
              f"{len(times)} timed steps")
    line = dict(metric="chunk_gdn2 fwd+bwd tokens/s/GPU (L=2048 Hk=12 Hv=24 K=V=128 bf16)", value=tok, unit="tokens/s",
                impl="reference", n_gpus=args.gpus, steps=len(times), warmup=args.warmup, ms_per_step=sec * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                config=dict(workload="chunk_gdn2 fwd+bwd B=1 L=2048 Hk=12 Hv=24 K=V=128 chunk=128 bf16"),
                cpu_baseline=dict(value=tok, unit="tokens/s", cores=cores, kind="port", sample=sample),
                e2e=dict(value=tok, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ main arm
# ------------------------------------------------------------------------------------------ long sequence
SPCFG = dict(L=131072, H=32, K=128, V=128, chunk=128)


def sp_leg(args, dn, dist, world, rank, dev):
    """KDA-style fwd+bwd on ONE packed sequence of 131072 tokens (channel-wise decay, per-head beta,
    documents of 2048..32768 tokens), split into equal contiguous shards over the ranks: the state
    chain crosses the ranks by NCCL point-to-point, everything else is local.  Total work is fixed, so
    this is strong scaling.  chunk_size is 128, the only size the reference's operator accepts."""
    from deltanet_b200 import sp
    c = SPCFG
    L, H, K, V = c["L"], c["H"], c["K"], c["V"]
    gen = torch.Generator().manual_seed(4000)
    lens, tot = [], 0
    while tot < L:
        n = int(torch.randint(2048, 32769, (1,), generator=gen))
        lens.append(min(n, L - tot))
        tot += lens[-1]
    seg = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32), torch.tensor(lens))[None]
    lo, hi = rank * L // world, (rank + 1) * L // world
    n = hi - lo
    g2 = torch.Generator(device=dev).manual_seed(4100 + rank)
    rn = lambda *sh: torch.randn(*sh, generator=g2, device=dev)
    q, k, v = (rn(1, n, H, K).bfloat16().requires_grad_(), rn(1, n, H, K).bfloat16().requires_grad_(),
               rn(1, n, H, V).bfloat16().requires_grad_())
    g = (-torch.exp(rn(1, n, H, K) * 0.39 - 1.0)).requires_grad_()
    beta = torch.sigmoid(rn(1, n, H)).requires_grad_()
    do = rn(1, n, H, V).bfloat16()
    seg_d = seg[:, lo:hi].contiguous().to(dev)

    def step():
        if world == 1:
            o = dn.chunk_kda(q, k, v, g, beta, segment_ids=seg_d, chunk_size=c["chunk"], qk_l2norm=True)
        else:
            o, _ = sp.chunk_gdn2_sp(q, k, v, g, beta, beta, segment_ids=seg_d, chunk_size=c["chunk"],
                                    precision="bf16", qk_l2norm=True)
        torch.autograd.grad(o, [q, k, v, g, beta], grad_outputs=do)

    steps = max(2, min(args.steps, 5))
    ms = time_steps(step, steps, 3, dist) / steps
    if rank == 0:
        print(json.dumps(dict(only="sp", metric="kda fwd+bwd tokens/s, one sequence split over the GPUs",
                              value=L / (ms * 1e-3), unit="tokens/s", n_gpus=world, steps=steps, warmup=3,
                              ms_per_step=ms, scaling="strong", dtype="bf16", data="synthetic",
                              config=dict(workload="chunk_kda fwd+bwd B=1 L=131072 H=32 K=V=128 chunk=128 bf16 "
                                                   "qk_l2norm, documents of 2048..32768 tokens",
                                          parallelism=f"sequence-sharded x{world}, state chain by NCCL send/recv"))),
              flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "chunk", "decode", "sp"],
                    help="profiling aid: run only the chunked fwd+bwd device loop, or only the decode loop")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod
    import deltanet_b200 as dn
    peaks = measured_peaks()
    tokens = CFG["B"] * CFG["L"]

    if args.only == "sp":
        sp_leg(args, dn, dist, world, rank, dev)
        return
    if args.only == "decode":
        dj = DecodeJob(DEC, dev, seed=3000 + rank, heads=DEC["Hv"] // world)
        ms_dec = time_steps(dj.step, args.steps, args.warmup, dist) / args.steps
        if rank == 0:
            print(json.dumps(dict(only="decode", us_per_step=ms_dec * 1e3,
                                  state_gbs=world * dj.state_bytes / (ms_dec * 1e-3) / 1e9)), flush=True)
        return
    # ---- device-resident throughput through the C ABI
    job = DeviceJob(CFG, dev, seed=1000 + rank)
    with ClockSampler(local) as clk:
        ms = time_steps(job.step, args.steps, args.warmup, dist)
    clocks = clk.summary()
    ms_step = ms / args.steps
    value = world * tokens / (ms_step * 1e-3)

    if args.only == "chunk":
        if rank == 0:
            print(json.dumps(dict(only="chunk", ms_per_step=ms_step, tokens_per_s=value)), flush=True)
        return
    # ---- per-kernel timing (each kernel alone, CUDA events on its stream) and the roofline of the slowest
    fl = alg_flops(CFG)
    items = CFG["B"] * job.ex.H * job.ex.NC
    job.step()
    per = {}
    for name in ("prepass_fwd", "state_fwd", "state_bwd", "prepass_bwd"):
        per[name] = time_steps(lambda: job.phase(name), 10, 3) / 10
    dom = max(per, key=per.get)
    by = alg_bytes(CFG)
    t_hbm = by[dom] * items / (peaks["hbm_gbs"] * 1e9)          # seconds at the measured copy bandwidth
    t_tc = fl[dom] * items / (peaks["bf16_tflops"] * 1e12)      # seconds at the measured dense bf16 rate
    sec = per[dom] * 1e-3
    if t_hbm >= t_tc:
        ach = by[dom] * items / sec / 1e9
        roofline = dict(kernel=dom, bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"])
    else:
        ach = fl[dom] * items / sec / 1e12
        roofline = dict(kernel=dom, bound="tensor", achieved=ach, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                        frac=ach / peaks["bf16_tflops"])
    roofline.update(traffic=NCU_DRAM_BYTES.get(dom), peak_source=peaks["source"],
                    tensor_frac=fl[dom] * items / sec / 1e12 / peaks["bf16_tflops"],
                    hbm_frac=by[dom] * items / sec / 1e9 / peaks["hbm_gbs"],
                    kernel_ms={k_: round(v_, 4) for k_, v_ in per.items()},
                    alg_gflop={k_: round(v_ * items / 1e9, 3) for k_, v_ in fl.items()},
                    alg_mbytes={k_: round(v_ * items / 1e6, 1) for k_, v_ in by.items()})

    # ---- end to end through the public operator with host buffers
    host = make_training_inputs(2000 + rank, CFG, pin=True)
    names = "qkvgbw"
    h2d = sum(host[n].numel() * host[n].element_size() for n in list(names) + ["do", "seg"])
    out_host = {n: torch.empty_like(host[n]).pin_memory() for n in list(names) + ["v"]}
    o_host = torch.empty_like(host["v"]).pin_memory()
    d2h = sum(host[n].numel() * host[n].element_size() for n in names) + o_host.numel() * o_host.element_size()

    def e2e_step():
        d = {n: host[n].to(dev, non_blocking=True) for n in list(names) + ["do", "seg"]}
        ins = [d[n].requires_grad_() for n in names]
        o = dn.chunk_gdn2(*ins, segment_ids=d["seg"], chunk_size=CFG["chunk"], precision="bf16", qk_l2norm=True)
        grads = torch.autograd.grad(o, ins, grad_outputs=d["do"])
        o_host.copy_(o.detach(), non_blocking=True)
        for n, gr in zip(names, grads):
            out_host[n].copy_(gr, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 40))
    ms_serial = time_steps(e2e_step, e2e_steps, 3, dist) / e2e_steps

    # The same work as a training loop would run it: batch i+1 is uploaded on a copy stream while
    # batch i computes and batch i-1's results are read back.  Every upload and read-back of the K
    # timed steps lies inside the timed region (run() starts and ends with all three streams joined).
    in_names = list(names) + ["do", "seg"]
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    slots = [{n: torch.empty_like(host[n], device=dev) for n in in_names} for _ in range(2)]
    loaded = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(freed[i % 2])
            for n in in_names:
                slots[i % 2][n].copy_(host[n], non_blocking=True)
            loaded[i % 2].record(s_in)

    def run_pipeline(k):
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        upload(0)
        for i in range(k):
            if i + 1 < k:
                upload(i + 1)
            d = slots[i % 2]
            main.wait_event(loaded[i % 2])
            ins = [d[n].detach().requires_grad_() for n in names]
            o = dn.chunk_gdn2(*ins, segment_ids=d["seg"], chunk_size=CFG["chunk"], precision="bf16", qk_l2norm=True)
            grads = torch.autograd.grad(o, ins, grad_outputs=d["do"])
            freed[i % 2].record(main)
            s_out.wait_stream(main)
            with torch.cuda.stream(s_out):
                o_host.copy_(o.detach(), non_blocking=True)
                o.record_stream(s_out)
                for n, gr in zip(names, grads):
                    out_host[n].copy_(gr, non_blocking=True)
                    gr.record_stream(s_out)
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    ms_e2e = time_steps(lambda: run_pipeline(e2e_steps), 1, 1, dist) / e2e_steps
    e2e = dict(value=world * tokens / (ms_e2e * 1e-3), unit="tokens/s", ms_per_step=ms_e2e,
               h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
               schedule="double-buffered: upload of batch i+1 and read-back of batch i-1 overlap batch i",
               unpipelined_ms_per_step=ms_serial)

    # ---- decode: value heads sharded over the ranks, no collective
    dj = DecodeJob(DEC, dev, seed=3000 + rank, heads=DEC["Hv"] // world)
    dsteps = 200
    ms_dec = time_steps(dj.step, dsteps, 20, dist) / dsteps
    st_gbs = world * dj.state_bytes / (ms_dec * 1e-3) / 1e9
    decode = dict(workload=f"gdn2 decode step, 256 sequences, Hk=16 Hv=32 K=V=128, bf16 state, {DEC['Hv'] // world} value heads per GPU",
                  us_per_step=ms_dec * 1e3, state_gbs=st_gbs,
                  total_gbs=world * (dj.state_bytes + dj.vec_bytes) / (ms_dec * 1e-3) / 1e9, steps=dsteps,
                  roofline=dict(bound="hbm", achieved=st_gbs / world, peak=peaks["hbm_gbs"], unit="GB/s",
                                frac=st_gbs / world / peaks["hbm_gbs"], traffic=None, peak_source=peaks["source"]))

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        cpu_oracle_step(CFG, 1.0 / 12.0)                       # warm-up on a small slice
        sec, f = cpu_oracle_step(CFG, 0.5)
        cpu = dict(value=tokens * f / sec, unit="tokens/s", cores=cores, kind="port",
                   sample=f"CPU oracle (port of the reference's chunked fwd+bwd), one step on {int(24 * f)} of 24 value "
                          f"heads at L=2048, {sec:.1f} s, token count scaled by the head fraction")
    line = dict(
        metric="chunk_gdn2 fwd+bwd tokens/s/GPU (L=2048 Hk=12 Hv=24 K=V=128 bf16)", value=value, unit="tokens/s",
        n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload="chunk_gdn2 fwd+bwd B=1 L=2048 Hk=12 Hv=24 K=V=128 chunk=128 precision=bf16 qk_l2norm "
                             "docs split at L/2 (per GPU)", global_batch=world, parallelism=f"batch-sharded x{world}, no collective",
                    l2=f"no flush: the step touches {job.bytes / 1e6:.0f} MB (inputs, residuals, scratch, grads) > 126 MB L2"),
        roofline=roofline, e2e=e2e, decode=decode, cpu_baseline=cpu,
        gpu_launches=(job.lib.dn_launch_count(job.shape, 0, 0) + job.lib.dn_launch_count(job.shape, 1, 0)) * args.steps,
        clocks=clocks)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
