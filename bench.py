#!/usr/bin/env python
"""Benchmark of the lrnnx scan hot path on B200 (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Default workload (benchmark configuration 1): the diagonal complex simplified scan used by
S5, complex64, B=8, P=256 states, H=512 channels, L=4096, forward + backward, recurrence
x_k = Lambda x_{k-1} + (B u)_k  (A = log Lambda, delta = 1, "dirac").

  value      tokens/s of the scan hot path (forward + backward kernels through the C ABI,
             captured once and replayed as CUDA graphs, operands resident in HBM); a token is
             one (batch, timestep) pair.  With N > 1
             every rank runs the full workload on its own batch shard (weak scaling) and the
             parameter gradients dA/dB/dC are all-reduced over NCCL inside the step.
  e2e        the same metric through the public op ``lrnnx_b200.ops.simplified_scan_fn``
             starting from pinned HOST tensors: host->device copies of the layer's real
             input x and of delta (micro-batched so the copies overlap the compute), the cast
             to complex on the device, the complex projections (cuBLAS), both scan kernels,
             and a device->host read of the loss every step.
  roofline   algorithmic HBM bytes of the dominant kernel / its mean launch time (CUDA
             events on the launching stream) against the measured copy bandwidth in
             MEASURED_PEAKS.json.
  cpu_baseline  the CPU oracle (a port of the reference's pure-PyTorch scan) timed on the
             host cores on a bounded sample of the same workload.

  workloads  the default run adds one sub-record per further workload (lm_cfg2: configs[2] LM training
             step; decode_cfg4: configs[4] generation; and the kernel-level ones below), each with
             its own ms_per_step, value, roofline, kernels, e2e and cpu_baseline (fewer steps each,
             so that the whole run stays within a few minutes): s6_cfg0 (configs[0]), s6_layer and
             s6_layer_f32 (one Mamba layer's scan at the configs[2] shape), s6_long (configs[3];
             sequence-parallel with a correctness check of the stitched output when N > 1),
             ssu_step (configs[4] state-update kernels), cauchy, s5_scan_zoh (configs[1] with a
             time-varying step size) and, when N > 1, s5_strong (configs[1] with its batch of 8
             split over the ranks: fixed total work).

``--impl reference`` times that CPU implementation alone (rank 0 only).
``--workload NAME`` runs one workload alone as the top-level line (no ``workloads`` key).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


# --------------------------------------------------------------------------- helpers
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured (sustained bf16 GEMM)"
    return 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            self.path = tempfile.NamedTemporaryFile(delete=False, suffix=".csv").name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in Path(self.path).read_text().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        # samples under load: the upper half of the clock samples (idle samples sit at low clocks)
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised in
# profiles/ (same workload, same kernel); None where no capture exists.
NCU_TRAFFIC = {
    ("s5_scan_cfg1", "simpscan_fwd_kernel"): 127.6e6,
    ("s5_scan_cfg1", "simpscan_bwd_kernel"): 301.5e6,
    ("s6_layer_cfg2", "selscan_fwd"): 223.4e6,
    ("s6_layer_cfg2", "selscan_bwd"): 382.2e6,
    ("cauchy_s4", "cauchy_fwd"): 76.1e6,
}


def cn(g, *shape):
    return torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g)) / math.sqrt(2)


def build_step_graphs(dev, copy_stream, issue_copies, compute):
    """Captures the two graphs of a double-buffered end-to-end step: graph s runs ``compute(s)`` on
    the capturing stream and, on a forked branch, ``issue_copies(s ^ 1)`` (the next step's
    host-to-device copies on ``copy_stream``).  Both slots are filled and ``compute`` is warmed up
    outside capture first."""
    cur = torch.cuda.current_stream()
    copy_stream.wait_stream(cur)
    issue_copies(0)
    issue_copies(1)
    cur.wait_stream(copy_stream)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        compute(0)
    cur.wait_stream(side)
    torch.cuda.synchronize()
    graphs = []
    for slot in range(2):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            c = torch.cuda.current_stream()
            copy_stream.wait_stream(c)
            issue_copies(slot ^ 1)
            compute(slot)
            c.wait_stream(copy_stream)
        graphs.append(g)
    return graphs


# --------------------------------------------------------------------------- workloads
class S5Scan:
    """benchmark configuration 1 (and its variants: time-varying step size, batch split over the ranks)."""
    dtype = "c64"
    metric, unit = "scan tokens/s (simplified scan fwd+bwd)", "tokens/s"

    def __init__(self, batch=8, P=256, H=512, L=4096, disc="dirac", name="s5_scan_cfg1", strong=False, cpu_full=True):
        self.batch, self.P, self.H, self.L, self.disc, self.name = batch, P, H, L, disc, name
        self.strong, self.cpu_full = strong, cpu_full
        self._set_sizes()

    def _set_sizes(self):
        batch, P, H, L = self.batch, self.P, self.H, self.L
        self.tokens = batch * L
        self.fwd_bytes = 20 * batch * P * L          # u 8 + delta 4 read, out 8 written per (b,p,l)
        self.bwd_bytes = 32 * batch * P * L          # u 8, delta 4, dout 8 read; du 8, ddelta 4 written
        step = "delta = 1" if self.disc == "dirac" else "time-varying delta"
        self.describe = {"workload": f"{self.name}: B={batch} P={P} H={H} L={L} complex64 {self.disc} ({step}) fwd+bwd",
                         "global_batch": batch, "seq_len": L, "states": P, "channels": H,
                         "l2": "operands of every kernel exceed the 126 MB L2 (fwd 168 MB, bwd 268 MB)"
                         if self.fwd_bytes > 1.3e8 else "L2 flushed by a 256 MB write between timed iterations"}
        self.flush = self.fwd_bytes <= 1.3e8

    def host_inputs(self, seed=0, batch=None, L=None):
        g = torch.Generator().manual_seed(seed)
        batch, L = batch or self.batch, L or self.L
        lam = torch.polar(0.9 + 0.099 * torch.rand(self.P, generator=g), math.pi / 10 * torch.rand(self.P, generator=g))
        A = torch.log(lam)
        B = cn(g, self.P, self.H) / math.sqrt(self.H)
        C = cn(g, self.H, self.P) / math.sqrt(self.P)
        u = torch.randn(batch, L, self.H, generator=g).transpose(1, 2).to(torch.complex64).contiguous()
        if self.disc == "dirac":
            delta = torch.ones(batch, self.P, L)
        else:      # the time-varying step sizes an LTV-S5 layer feeds (lrnnx/models/ltv/s5.py:113-115)
            delta = 0.5 + torch.rand(batch, self.P, L, generator=g)
        gout = cn(g, batch, self.H, L)
        return dict(u=u, delta=delta, A=A, B=B, C=C, gout=gout)

    def setup(self, dev, pg):
        from lrnnx_b200 import simplified_scan_cuda
        from lrnnx_b200.ops import simplified_scan_fn
        self.dev, self.pg = dev, pg
        if self.strong and pg is not None:
            # fixed total work: the batch of 8 rows is split over the ranks (batch x state rows are
            # independent recurrences; only dA is reduced)
            w = torch.distributed.get_world_size()
            self.batch = max(1, self.batch // w)
            self._set_sizes()
            self.scaling = "strong"
            self.describe["parallelism"] = f"batch of {self.batch * w} split over {w} GPUs ({self.batch} per GPU)"
            self.describe["global_batch"] = self.batch * w
        h = self.host_inputs()
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if self.flush else None
        self.h_x = h["u"].real.transpose(1, 2).contiguous().pin_memory()      # (batch, L, H) float32: the layer's input
        self.h_delta, self.h_gout = h["delta"].pin_memory(), h["gout"].pin_memory()
        self.A, self.B, self.C = (h[k].to(dev) for k in ("A", "B", "C"))
        self.u, self.delta, self.gout = h["u"].to(dev), self.h_delta.to(dev), self.h_gout.to(dev)
        self.copy_stream = torch.cuda.Stream(device=dev)
        # kernel-level operands (what SimplifiedScanFn hands to the extension)
        self.Bu = torch.einsum("ph,bhl->bpl", self.B, self.u).contiguous()
        self.dBu_in = torch.einsum("hp,bhl->bpl", self.C.conj(), self.gout).contiguous()
        self.A_k = self.A.unsqueeze(-1).contiguous()
        self.one = torch.ones(self.P, 1, dtype=torch.complex64, device=dev)
        self.ext, self.op = simplified_scan_cuda, simplified_scan_fn
        self.ev = []
        self._work = None
        self._ar_buf = torch.zeros(self.P, 1, 2, device=dev)
        # The two extension calls are captured once as CUDA graphs (after a warm-up on a side
        # stream); a step replays them, so the timed region holds the kernels and not the
        # Python / ctypes launch path.
        args = (self.Bu, self.delta, self.A_k, self.one, self.one, None)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                out, x = self.ext.fwd(*args, self.disc)
                self.ext.bwd(*args, self.dBu_in, x, self.disc, need_dB_dC=False, out_=out)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.g_fwd, self.g_bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.g_fwd):
            self.out, self.x = self.ext.fwd(*args, self.disc)
        with torch.cuda.graph(self.g_bwd):
            # as SimplifiedScanFn.backward calls it (identity B and C: dB / dC are not needed, and the
            # forward output, which is the state sequence, is handed back)
            self.res = self.ext.bwd(*args, self.dBu_in, self.x, self.disc, need_dB_dC=False, out_=self.out)
        self.g_step = None
        if pg is not None:
            # Data-parallel step as ONE graph per parity: forward, backward and the copy of dA into
            # buffer p on the main branch; the all-reduce of the previous step's dA (buffer 1 - p) on a
            # forked branch, so the collective overlaps this step's kernels and costs no host work per
            # step (no stream wait, no enqueue: one graph launch).
            try:
                self._ar = [torch.zeros(self.P, 1, 2, device=dev) for _ in range(2)]
                for buf in self._ar:
                    torch.distributed.all_reduce(buf, group=pg)          # communicator warm-up outside capture
                torch.cuda.synchronize()
                graphs = []
                for par in range(2):
                    g = torch.cuda.CUDAGraph()
                    branch = torch.cuda.Stream(device=dev)
                    with torch.cuda.graph(g):
                        branch.wait_stream(torch.cuda.current_stream())
                        with torch.cuda.stream(branch):
                            torch.distributed.all_reduce(self._ar[1 - par], group=pg)
                        out, x = self.ext.fwd(*args, self.disc)
                        res = self.ext.bwd(*args, self.dBu_in, x, self.disc, need_dB_dC=False, out_=out)
                        self._ar[par].copy_(torch.view_as_real(res[2]))
                        torch.cuda.current_stream().wait_stream(branch)
                    graphs.append(g)
                self.g_step, self._parity = graphs, 0
                self.describe["collective"] = "dA all-reduce (NCCL) captured in the step's CUDA graph on a forked branch"
            except Exception as exc:      # capture of the collective refused: per-step asynchronous all-reduce instead
                self.g_step = None
                self.describe["collective"] = f"dA all-reduce (NCCL) enqueued per step ({type(exc).__name__} during graph capture)"
                torch.cuda.synchronize()

    def step(self, record=False):
        """forward + backward scan kernels through the extension entry points (graph replay)."""
        if self.g_step is not None:
            self.g_step[self._parity].replay()
            self._parity ^= 1
            return self.res
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            e[0].record()
        self.g_fwd.replay()
        if record:
            e[1].record()
        self.g_bwd.replay()
        if record:
            e[2].record()
            self.ev.append(e)
        if self.pg is not None:
            # Data-parallel reduction of the parameter gradient, overlapped with the next step's kernels
            # as a gradient all-reduce is in training: dA is copied to a side buffer and reduced
            # asynchronously on NCCL's stream; the buffer is reused once the previous reduction is done.
            if self._work is not None:
                self._work.wait()
            self._ar_buf.copy_(torch.view_as_real(self.res[2]))
            self._work = torch.distributed.all_reduce(self._ar_buf, group=self.pg, async_op=True)
        return self.res

    launches_per_step = 2

    def drain(self):
        if self.g_step is not None:
            # the dA of the last step is still to be reduced
            torch.distributed.all_reduce(self._ar[self._parity ^ 1], group=self.pg)
            return
        if self._work is not None:
            self._work.wait()
            self._work = None

    e2e_micro_batches = 4

    def _issue_copies(self, slot):
        """Enqueue the host-to-device copies of one step's inputs on the copy stream into staging
        slot ``slot``."""
        with torch.cuda.stream(self.copy_stream):
            self._stage_x[slot].copy_(self.h_x, non_blocking=True)
            self._stage_delta[slot].copy_(self.h_delta, non_blocking=True)

    def _e2e_compute(self, slot):
        """Forward + backward of simplified_scan_fn over the micro-batches of staging slot ``slot``."""
        n = self.e2e_micro_batches if self.batch % self.e2e_micro_batches == 0 else 1
        mb = self.batch // n
        A, B, C = self._e2e_leaves
        for t in (A, B, C):
            t.grad = None
        d_x, d_delta = self._stage_x[slot], self._stage_delta[slot]
        total = torch.zeros((), device=self.dev)
        for i in range(n):
            sl = slice(i * mb, (i + 1) * mb)
            u = d_x[sl].transpose(1, 2).contiguous().to(torch.complex64).requires_grad_(True)
            delta = d_delta[sl].detach().requires_grad_(True)
            y = self.op(u, delta, A, B, C, discretization=self.disc)
            loss = (y * self.gout[sl].conj()).real.sum()
            loss.backward()
            total += loss.detach()
        self._e2e_total.copy_(total)

    def _e2e_build(self):
        """Staging buffers and the two step graphs.  Graph s computes from staging slot s while, on a
        forked branch, the copy stream brings the next step's inputs from pinned host memory into
        slot s ^ 1 (a data loader's prefetch): every step issues one full copy of the inputs (100 MB),
        the copies overlap the compute, and a step costs the host one graph launch."""
        self._stage_x = [torch.empty_like(self.h_x, device=self.dev) for _ in range(2)]
        self._stage_delta = [torch.empty_like(self.h_delta, device=self.dev) for _ in range(2)]
        self._e2e_leaves = tuple(t.detach().clone().requires_grad_(True) for t in (self.A, self.B, self.C))
        self._e2e_total = torch.zeros((), device=self.dev)
        self._e2e_graphs = build_step_graphs(self.dev, self.copy_stream, self._issue_copies, self._e2e_compute)
        # the first replay computes from slot 0, which the copies above have filled
        self._slot = 0

    def e2e_step(self):
        """One step as the LTV-S5 layer drives the op (lrnnx/models/ltv/s5.py:111-112): the real
        input x (batch, L, H) and delta arrive from pinned host memory, u = x^T cast to complex64
        on the device, then simplified_scan_fn forward + backward in micro-batches (parameter
        gradients accumulate over them), and the loss is read back.  The step is replayed from a
        CUDA graph (see ``_e2e_build``)."""
        if getattr(self, "_e2e_graphs", None) is None:
            try:
                self._e2e_build()
                self.describe["e2e"] = "step replayed from a CUDA graph; next step's inputs prefetched on a forked branch"
            except Exception as exc:      # capture refused: the same step enqueued from the host
                torch.cuda.synchronize()
                self._e2e_graphs = False
                self.describe["e2e"] = f"step enqueued from the host ({type(exc).__name__} during graph capture)"
        if self._e2e_graphs:
            self._e2e_graphs[self._slot].replay()
            self._slot ^= 1
        else:
            cur = torch.cuda.current_stream()
            self.copy_stream.wait_stream(cur)
            self._issue_copies(0)
            cur.wait_stream(self.copy_stream)
            self._e2e_compute(0)
        if self.pg is not None:
            for t in self._e2e_leaves:
                torch.distributed.all_reduce(torch.view_as_real(t.grad), group=self.pg)
        return float(self._e2e_total.item())

    def e2e_bytes(self):
        return self.h_x.numel() * 4 + self.h_delta.numel() * 4, 4

    def kernel_rooflines(self):
        if not self.ev:      # the step ran as one graph: time the two kernels apart in a short pass of their own
            for _ in range(8):
                e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                if self.flush_buf is not None:
                    self.flush_buf.zero_()
                e[0].record()
                self.g_fwd.replay()
                e[1].record()
                self.g_bwd.replay()
                e[2].record()
                self.ev.append(e)
            torch.cuda.synchronize()
            self.ev = self.ev[3:]
        f = [a[0].elapsed_time(a[1]) for a in self.ev]
        b = [a[1].elapsed_time(a[2]) for a in self.ev]
        return {"simpscan_fwd_kernel": (self.fwd_bytes, statistics.mean(f)),
                "simpscan_bwd_kernel": (self.bwd_bytes, statistics.mean(b))}

    # CPU arm: the full workload for the headline line; batch 1 and the first 1024 steps (same P
    # and H: the work per token is unchanged) for the sub-records
    @property
    def cpu_sample(self):
        if self.cpu_full:
            return f"the full workload: batch {self.batch}, {self.L} timesteps, P={self.P}, H={self.H}"
        return f"batch 1, first 1024 of {self.L} timesteps, P={self.P}, H={self.H}"

    def cpu_step(self):
        from oracle import scan_oracle as O
        cb, cl = (self.batch, self.L) if self.cpu_full else (1, min(self.L, 1024))
        if not hasattr(self, "_cpu"):
            self._cpu = self.host_inputs(batch=cb, L=cl)
        h = self._cpu
        leaves = [h[k].clone().requires_grad_(True) for k in ("u", "delta", "A", "B", "C")]
        y = O.simplified_scan_oracle(*leaves, discretization=self.disc)
        torch.autograd.grad(y, leaves, h["gout"])
        return cb * cl


class S6Scan:
    """Selective scan (S6/Mamba) forward(+backward); shapes of benchmark configurations 0, 2 (one layer) and 3."""
    roofline_note = ("with dstate 16 the scan needs one ex2 and ~7 fp32 operations per (timestep, state, channel) "
                     "for 4-10 bytes: it is bound by fp32 / SFU instruction issue, not by HBM (ncu: 62 % of the issue "
                     "slots busy in the forward, DRAM below 10 %)")
    metric, unit = "scan tokens/s (selective scan)", "tokens/s"

    def __init__(self, name, batch, dim, L, N, dtype, backward=True):
        self.name, self.batch, self.dim, self.L, self.N, self.tdtype, self.backward = name, batch, dim, L, N, dtype, backward
        self.dtype = "f32" if dtype == torch.float32 else "bf16 i/o, f32 state"
        s = 4 if dtype == torch.float32 else 2
        bdl, bnl = batch * dim * L, batch * N * L
        self.tokens = batch * L
        self.fwd_bytes = 5 * s * bdl + 2 * s * bnl
        self.bwd_bytes = 8 * s * bdl + (2 * s + 8) * bnl
        self.describe = {"workload": f"{name}: B={batch} D={dim} L={L} N={N} {self.dtype} "
                                     f"{'fwd+bwd' if backward else 'fwd'} mamba, z, D, delta_bias, softplus",
                         "global_batch": batch, "seq_len": L,
                         "l2": "L2 flushed by a 256 MB write between timed iterations" if self.fwd_bytes < 2.6e8
                         else "operands exceed the 126 MB L2"}
        self.flush = self.fwd_bytes < 2.6e8
        self.launches_per_step = 2 if backward else 1

    def host_inputs(self, seed=0, dim=None, L=None):
        g = torch.Generator().manual_seed(seed)
        batch, dim, L, N = self.batch, dim or self.dim, L or self.L, self.N
        dt = torch.exp(torch.rand(dim, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
        return dict(u=torch.randn(batch, dim, L, generator=g).to(self.tdtype),
                    delta=torch.randn(batch, dim, L, generator=g).to(self.tdtype),
                    A=-torch.arange(1, N + 1, dtype=torch.float32).repeat(dim, 1),
                    B=torch.randn(batch, 1, N, L, generator=g).to(self.tdtype),
                    C=torch.randn(batch, 1, N, L, generator=g).to(self.tdtype),
                    D=torch.ones(dim), z=torch.randn(batch, dim, L, generator=g).to(self.tdtype),
                    delta_bias=dt + torch.log(-torch.expm1(-dt)),
                    gout=torch.randn(batch, dim, L, generator=g).to(self.tdtype))

    def setup(self, dev, pg):
        from lrnnx_b200 import selective_scan_cuda
        from lrnnx_b200.ops import selective_scan_fn
        self.dev, self.pg, self.ext, self.op = dev, pg, selective_scan_cuda, selective_scan_fn
        h = self.host_inputs()
        # the long forward-only configuration runs sequence-parallel on N > 1 GPUs: every rank keeps
        # its slice of the sequence (fixed total work: strong scaling)
        self.sp = pg is not None and not self.backward
        if self.sp:
            import torch.distributed as dist
            from lrnnx_b200.sp import sp_selective_scan_fwd
            self.sp_fwd = sp_selective_scan_fwd
            self.scaling = "strong"
            r, w = dist.get_rank(), dist.get_world_size()
            lo, hi = (r * self.L // w) // 8 * 8, ((r + 1) * self.L // w) // 8 * 8 if r + 1 < w else self.L
            if r == 0:   # 16 channels over the full sequence, for the check of the stitched result
                self._chk = {k: (v[:, :16].clone() if v.dim() == 3 else (v.clone() if v.dim() == 4 else v[:16].clone()))
                             for k, v in h.items()}
            h = {k: (v[..., lo:hi].contiguous() if v.dim() >= 3 else v) for k, v in h.items()}
            self.describe["parallelism"] = f"sequence-parallel over {w} GPUs: chunk-state all-gather + fix-up"
            self.fwd_bytes //= w
        self.h = {k: v.pin_memory() for k, v in h.items()}
        self.t = {k: v.to(dev) for k, v in h.items()}
        self.ev = []
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if self.flush else None
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.g_fwd = self.g_bwd = None
        if not self.sp:
            # the extension calls are captured once as CUDA graphs (after a warm-up on a side stream);
            # a step replays them, so the timed region holds the kernels and not the Python launch path
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._call_fwd()
                    if self.backward:
                        self._call_bwd()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.g_fwd = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g_fwd):
                self._call_fwd()
            if self.backward:
                self.g_bwd = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.g_bwd):
                    self._call_bwd()

    def _call_fwd(self):
        t = self.t
        self.fwd_out = self.ext.fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["z"], t["delta_bias"],
                                    None, True, "mamba")

    def _call_bwd(self):
        t = self.t
        out, x, _ = self.fwd_out
        self.bwd_out = self.ext.bwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["z"], t["delta_bias"], None,
                                    t["gout"], x, out, None, True, False, "mamba")

    def step(self, record=False):
        t = self.t
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            e[0].record()
        if self.g_fwd is not None:
            self.g_fwd.replay()
            if record:
                e[1].record()
            if self.g_bwd is not None:
                self.g_bwd.replay()
            if record:
                e[2].record()
                self.ev.append(e)
            if self.pg is not None and self.backward:
                torch.distributed.all_reduce(self.bwd_out[2], group=self.pg)
            return self.bwd_out if self.backward else None
        if self.sp:
            self.sp_fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["z"], t["delta_bias"], True, self.pg)
            if record:
                e[1].record()
                e[2].record()
                self.ev.append(e)
            return None
        out, x, out_z = self.ext.fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["z"], t["delta_bias"],
                                     None, True, "mamba")
        if record:
            e[1].record()
        res = None
        if self.backward:
            res = self.ext.bwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["z"], t["delta_bias"], None,
                               t["gout"], x, out, None, True, False, "mamba")
        if record:
            e[2].record()
            self.ev.append(e)
        if self.pg is not None and res is not None:
            torch.distributed.all_reduce(res[2], group=self.pg)
        return res

    def sp_check(self):
        """Sequence-parallel run only: the stitched gated output of 16 channels, gathered from all
        ranks, against the unsplit forward of those channels on rank 0.  Returns the record on
        rank 0 (None elsewhere)."""
        import torch.distributed as dist
        t = self.t
        y, _ = self.sp_fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["z"], t["delta_bias"], True, self.pg)
        mine = y[:, :16].contiguous()
        parts = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(parts, mine, group=self.pg)
        if dist.get_rank() != 0:
            return None
        c = {k: v.to(self.dev) for k, v in self._chk.items()}
        ref = self.ext.fwd(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"], None, True,
                           "mamba")[2].float()
        got = torch.cat(parts, dim=-1).float()
        scale = float(ref.abs().max())
        err = (got - ref).abs()
        ok = bool((err <= 1e-2 * scale + 3e-2 * ref.abs()).all())
        return {"channels": 16, "max_abs_err": float(err.max()), "max_rel_err": float(err.max()) / scale, "ok": ok,
                "tolerance": "|d| <= 1e-2 max|ref| + 3e-2 |ref| (bf16 outputs)"}

    _e2e_names = ("u", "delta", "B", "C", "z")

    def _issue_copies(self, slot):
        with torch.cuda.stream(self.copy_stream):
            for k in self._e2e_names:
                self._stage[slot][k].copy_(self.h[k], non_blocking=True)

    def _e2e_compute(self, slot):
        """selective_scan_fn forward (+ backward) on staging slot ``slot``, in micro-batches when the
        batch allows (parameter gradients accumulate over them); the loss goes to a static scalar."""
        n = 4 if self.batch % 4 == 0 else 1
        mb = self.batch // n
        st = self._stage[slot]
        A, D, bias = self._e2e_leaves
        for t in (A, D, bias):
            t.grad = None
        total = torch.zeros((), device=self.dev)
        for i in range(n):
            sl = slice(i * mb, (i + 1) * mb)
            lv = {k: st[k][sl].detach().requires_grad_(self.backward) for k in self._e2e_names}
            y = self.op(lv["u"], lv["delta"], A, lv["B"], lv["C"], D, lv["z"], bias, delta_softplus=True,
                        discretization="mamba")
            loss = (y.float() * self.t["gout"][sl].float()).sum()
            if self.backward:
                loss.backward()
            total += loss.detach()
        self._e2e_total.copy_(total)

    def _e2e_build(self):
        """Two staging slots and two step graphs: graph s computes from slot s while a forked branch
        copies the next step's inputs from pinned host memory into slot s ^ 1."""
        self._stage = [{k: torch.empty_like(self.t[k]) for k in self._e2e_names} for _ in range(2)]
        self._e2e_leaves = tuple(self.t[k].detach().clone().requires_grad_(self.backward) for k in ("A", "D", "delta_bias"))
        self._e2e_total = torch.zeros((), device=self.dev)
        self._e2e_graphs = build_step_graphs(self.dev, self.copy_stream, self._issue_copies, self._e2e_compute)
        self._slot = 0

    def e2e_step(self):
        """One step through the public op with the inputs arriving from pinned host memory and the
        loss read back.  The sequence-parallel case enqueues from the host (its exchange is a
        collective plus host-side folding); everything else replays a CUDA graph per step."""
        if self.sp:
            t = {k: (self.t[k].copy_(self.h[k], non_blocking=True)) for k in self._e2e_names}
            y, _ = self.sp_fwd(t["u"], t["delta"], self.t["A"], t["B"], t["C"], self.t["D"], t["z"],
                               self.t["delta_bias"], True, self.pg)
            return float((y.float() * self.t["gout"].float()).sum().item())
        if getattr(self, "_e2e_graphs", None) is None:
            if self.fwd_bytes > 2e9:            # config 3: the copies are the step; no second staging set
                self._e2e_graphs = False
            else:
                try:
                    self._e2e_build()
                    self.describe["e2e"] = "step replayed from a CUDA graph; next step's inputs prefetched on a forked branch"
                except Exception as exc:
                    torch.cuda.synchronize()
                    self._e2e_graphs = False
                    self.describe["e2e"] = f"step enqueued from the host ({type(exc).__name__} during graph capture)"
        if self._e2e_graphs:
            self._e2e_graphs[self._slot].replay()
            self._slot ^= 1
        else:
            if getattr(self, "_stage", None) is None:
                self._stage = [{k: self.t[k] for k in self._e2e_names}]
                self._e2e_leaves = tuple(self.t[k].detach().clone().requires_grad_(self.backward)
                                         for k in ("A", "D", "delta_bias"))
                self._e2e_total = torch.zeros((), device=self.dev)
            cur = torch.cuda.current_stream()
            self.copy_stream.wait_stream(cur)
            self._issue_copies(0)
            cur.wait_stream(self.copy_stream)
            self._e2e_compute(0)
        if self.pg is not None and self.backward:
            torch.distributed.all_reduce(self._e2e_leaves[0].grad, group=self.pg)
        return float(self._e2e_total.item())

    def e2e_bytes(self):
        return sum(self.h[k].numel() * self.h[k].element_size() for k in ("u", "delta", "B", "C", "z")), 4

    def kernel_rooflines(self):
        f = [a[0].elapsed_time(a[1]) for a in self.ev]
        r = {"selscan_fwd": (self.fwd_bytes, statistics.mean(f))}
        if self.backward:
            b = [a[1].elapsed_time(a[2]) for a in self.ev]
            r["selscan_bwd"] = (self.bwd_bytes, statistics.mean(b))
        return r

    @property
    def cpu_sample(self):
        return f"{self._cpu_dim} of {self.dim} channels, first {self._cpu_L} of {self.L} timesteps, all batches"

    def cpu_step(self):
        from oracle import scan_oracle as O
        self._cpu_dim, self._cpu_L = min(self.dim, 64), min(self.L, 1024)
        if not hasattr(self, "_cpu"):
            self._cpu = self.host_inputs(dim=self._cpu_dim, L=self._cpu_L)
        h = self._cpu
        names = ("u", "delta", "A", "B", "C", "D", "z", "delta_bias")
        leaves = {k: h[k].clone().requires_grad_(self.backward) for k in names}
        y = O.selective_scan_oracle(**leaves, delta_softplus=True, discretization="mamba")
        if self.backward:
            torch.autograd.grad(y, list(leaves.values()), h["gout"])
        # tokens of the sample scaled by the channel fraction (channels are independent rows)
        return self.batch * self._cpu_L * self._cpu_dim / self.dim


class SsuStep:
    """Decode step kernel at the benchmark configuration 4 shape: 48 layers x selective_state_update with
    batch 64, d_inner 4096, dstate 16, bf16 activations, fp32 state (one step = 48 launches; the
    projections, conv and norms of the model are outside the path)."""
    name = "ssu_step_cfg4"
    dtype = "bf16 i/o, f32 state"
    metric, unit = "generated tokens/s (state-update kernels only)", "tokens/s"
    launches_per_step = 48
    cpu_sample = "2 of 48 layers, full batch"

    def __init__(self, batch=64, dim=4096, N=16, layers=48):
        self.batch, self.dim, self.N, self.layers = batch, dim, N, layers
        self.tokens = batch
        per_layer = 2 * batch * dim * N * 4 + 4 * batch * dim * 2 + 2 * batch * N * 2 + 4 * dim * N + 8 * dim
        self.fwd_bytes = per_layer
        self.describe = {"workload": f"{self.name}: {layers} layers, batch {batch}, d_inner {dim}, dstate {N}",
                         "global_batch": batch, "seq_len": 1, "launch": "CUDA graph replay of the 48 launches",
                         "l2": "48 layer states (805 MB) cycle through the 126 MB L2"}

    def _layer(self, g, batch=None):
        b = batch or self.batch
        r = lambda *s: torch.randn(*s, generator=g)
        return dict(state=r(b, self.dim, self.N), x=r(b, self.dim).bfloat16(), dt=r(b, self.dim).bfloat16(),
                    A=-torch.rand(self.dim, self.N, generator=g) - 0.5, B=r(b, self.N).bfloat16(),
                    C=r(b, self.N).bfloat16(), D=r(self.dim), z=r(b, self.dim).bfloat16(),
                    dt_bias=torch.rand(self.dim, generator=g) - 4.0)

    def setup(self, dev, pg):
        from lrnnx_b200.ops import selective_state_update
        self.op, self.pg = selective_state_update, pg
        g = torch.Generator().manual_seed(0)
        self.layers_t = [{k: v.to(dev) for k, v in self._layer(g).items()} for _ in range(self.layers)]
        self.h_x = self.layers_t[0]["x"].cpu().pin_memory()
        self.ev = []
        # the decode path replays a captured CUDA graph (warm-up on a side stream, then capture),
        # the pattern of lrnnx/utils/generation.py:143-155
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self._eager()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = self._eager()

    def _eager(self):
        for t in self.layers_t:
            out = self.op(t["state"], t["x"], t["dt"], t["A"], t["B"], t["C"], t["D"], t["z"], t["dt_bias"], True)
        return out

    def step(self, record=False):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(2)] if record else None
        if record:
            e[0].record()
        self.graph.replay()
        if record:
            e[1].record()
            self.ev.append(e)
        return self.out

    def e2e_step(self):
        self.layers_t[0]["x"].copy_(self.h_x, non_blocking=True)
        out = self.step()
        return float(out.float().sum().item())

    def e2e_bytes(self):
        return self.h_x.numel() * 2, 4

    def kernel_rooflines(self):
        ms = statistics.mean(a[0].elapsed_time(a[1]) for a in self.ev) / self.layers
        return {"ssu_tma_kernel": (self.fwd_bytes, ms)}

    def cpu_step(self):
        from oracle import scan_oracle as O
        if not hasattr(self, "_cpu"):
            g = torch.Generator().manual_seed(0)
            self._cpu = [self._layer(g) for _ in range(2)]
        for t in self._cpu:
            a = {k: (v.float() if v.dtype == torch.bfloat16 else v) for k, v in t.items() if k != "state"}
            O.selective_state_update_oracle(t["state"], **a, dt_softplus=True)
        return self.batch * 2 / self.layers


class CauchyKernel:
    """S4 kernel generation: the symmetric Cauchy multiply at the shape of the reference's
    micro-benchmark (benchmarks/benchmark_cauchy.py:49-51): 1024 rows, 32 conjugate-pair poles,
    16384 frequencies, complex64, forward + backward.  A unit is one output element (row,
    frequency).  The kernel is bound by the fp32 pipe (two complex reciprocals per
    (row, frequency, pole)), not by HBM; the HBM fraction is reported for completeness."""
    name = "cauchy_s4"
    roofline_note = "bound by the fp32 pipe (two complex reciprocals per (row, frequency, pole)), not by HBM"
    dtype = "c64"
    metric, unit = "Cauchy output elements/s (fwd+bwd)", "elements/s"
    launches_per_step = 3      # forward, backward partials, backward fold

    def __init__(self, rows=1024, n=32, L=16384):
        self.rows, self.n, self.L = rows, n, L
        self.tokens = rows * L
        self.fwd_bytes = 16 * rows * n + 8 * L + 8 * rows * L            # v, w, z read; out written
        self.bwd_bytes = 16 * rows * n + 8 * L + 8 * rows * L + 16 * rows * n   # + dout read, dv, dw written
        self.describe = {"workload": f"{self.name}: rows={rows} pole pairs={n} L={L} complex64 fwd+bwd",
                         "l2": "a 256 MB write flushes the 126 MB L2 before every step"}

    def host_inputs(self, rows=None, L=None):
        g = torch.Generator().manual_seed(2357)
        rows, L = rows or self.rows, L or self.L
        return dict(v=cn(g, rows, self.n), w=cn(g, rows, self.n) - 1.0,
                    z=torch.polar(torch.ones(L), torch.randn(L, generator=g)), gout=cn(g, rows, L))

    def setup(self, dev, pg):
        from lrnnx_b200 import structured_kernels
        from lrnnx_b200.ops import cauchy_mult
        self.dev, self.pg, self.ext, self.op = dev, pg, structured_kernels, cauchy_mult
        self.h = {k: v.pin_memory() for k, v in self.host_inputs().items()}
        self.t = {k: v.to(dev) for k, v in self.h.items()}
        self.ev = []
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step(self, record=False):
        t = self.t
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            e[0].record()
        self.ext.cauchy_mult_sym_fwd(t["v"], t["z"], t["w"])
        if record:
            e[1].record()
        res = self.ext.cauchy_mult_sym_bwd(t["v"], t["z"], t["w"], t["gout"])
        if record:
            e[2].record()
            self.ev.append(e)
        return res

    def e2e_step(self):
        v, w = (self.t[k].copy_(self.h[k], non_blocking=True).detach().requires_grad_(True) for k in ("v", "w"))
        z = self.t["z"].copy_(self.h["z"], non_blocking=True)
        y = self.op(v, z, w)
        torch.autograd.backward(y, self.t["gout"])
        return float(torch.view_as_real(v.grad).sum().item())

    def e2e_bytes(self):
        return sum(self.h[k].numel() * 8 for k in ("v", "w", "z")), 4

    # fp32 operations per (row, frequency, pole pair): two terms v / (z - w), each a complex
    # subtraction (2), |d|^2 (3), a reciprocal (1), two scalings (2), a complex product (6) and a
    # complex accumulation (2); the backward evaluates 1/d and 1/d^2 terms for dv and dw: twice that
    FLOP_FWD, FLOP_BWD = 32, 64

    def kernel_rooflines(self):
        f = [a[0].elapsed_time(a[1]) for a in self.ev]
        b = [a[1].elapsed_time(a[2]) for a in self.ev]
        terms = self.rows * self.L * self.n
        return {"cauchy_fwd": (self.fwd_bytes, statistics.mean(f), {"flops": self.FLOP_FWD * terms}),
                "cauchy_bwd": (self.bwd_bytes, statistics.mean(b), {"flops": self.FLOP_BWD * terms})}

    cpu_sample = "64 of 1024 rows, all 16384 frequencies"

    def cpu_step(self):
        from oracle import scan_oracle as O
        if not hasattr(self, "_cpu"):
            self._cpu = self.host_inputs(rows=64)
        h = self._cpu
        v, w = (h[k].clone().requires_grad_(True) for k in ("v", "w"))
        y = O.cauchy_oracle(v, h["z"], w, compute_dtype=torch.complex64)
        torch.autograd.grad(y, [v, w], h["gout"])
        return 64 * self.L


class BlockKernels:
    """The HBM-bound kernels around the scan in a Mamba block and LM step, at the config-2 shapes:
    causal convolution + SiLU forward / backward on (8, 1536, 2048) bf16, residual add + RMSNorm
    forward / backward on (16384, 768) bf16, next-token cross-entropy forward / backward on
    (16384, 50280) bf16 logits, and the narrow projection of a decoding step (64 x 4096 -> 160).
    A step runs each REPEAT times (one CUDA graph per kernel); a token is one (batch, position) of the
    config-2 batch, counted once per repeat."""
    name = "block_kernels_cfg2"
    dtype = "bf16"
    metric, unit = "tokens/s through the block kernels (conv, norm, loss; fwd+bwd)", "tokens/s"
    launches_per_step = 7 * 4
    roofline_note = ("conv and norm operands (25-50 MB per tensor) partly stay in the 126 MB L2 between the forward and "
                     "backward launch, as they do inside the LM step; the fraction is algorithmic bytes over time")

    def __init__(self, batch=8, d_inner=1536, L=2048, d_model=768, vocab=50280):
        self.batch, self.d_inner, self.L, self.d_model, self.vocab = batch, d_inner, L, d_model, vocab
        self.tokens = batch * L * self.REPEAT
        self.describe = {"workload": f"{self.name}: conv (8,{d_inner},{L}), norm ({batch * L},{d_model}), "
                                     f"loss ({batch * L},{vocab}), x_proj 64x4096->160; bf16",
                         "global_batch": batch, "seq_len": L,
                         "l2": "the loss kernels stream 1.65 GB of logits; a 256 MB write flushes the L2 before every step"}

    def setup(self, dev, pg):
        from lrnnx_b200.ops.cross_entropy import cross_entropy
        from lrnnx_b200.ops.linear_step import linear_step
        from lrnnx_b200.ops.mamba_block import causal_conv1d_fn, rms_norm_fn
        self.dev, self.pg = dev, pg
        self.fn = dict(conv=causal_conv1d_fn, norm=rms_norm_fn, xent=cross_entropy, lin=linear_step)
        g = torch.Generator().manual_seed(0)
        bf = torch.bfloat16
        rows = self.batch * self.L
        mk = lambda *s: torch.randn(*s, generator=g).to(bf)
        self.h_x = mk(self.batch, self.d_inner, self.L).pin_memory()
        self.t = dict(x=self.h_x.to(dev).requires_grad_(True), w=mk(self.d_inner, 4).to(dev).requires_grad_(True),
                      b=torch.zeros(self.d_inner, dtype=bf, device=dev, requires_grad=True),
                      gconv=mk(self.batch, self.d_inner, self.L).to(dev),
                      h=mk(rows, self.d_model).to(dev).requires_grad_(True), r=mk(rows, self.d_model).to(dev).requires_grad_(True),
                      g=torch.ones(self.d_model, dtype=bf, device=dev, requires_grad=True), gnorm=mk(rows, self.d_model).to(dev),
                      logits=mk(rows, self.vocab).to(dev).requires_grad_(True),
                      labels=torch.randint(0, self.vocab, (rows,), generator=g).to(dev),
                      xs=mk(64, 4096).to(dev), wx=(mk(160, 4096) / 64).to(dev))
        self.ev = []
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        s2 = 2
        BDL, RC, RV = self.batch * self.d_inner * self.L, rows * self.d_model, rows * self.vocab
        self.bytes = {"conv1d_fwd": 2 * BDL * s2, "conv1d_bwd": 3 * BDL * s2, "rmsnorm_fwd": 4 * RC * s2,
                      "rmsnorm_bwd": 4 * RC * s2, "xent_fwd": RV * s2, "xent_bwd": 2 * RV * s2,
                      "skinny_linear": 160 * 4096 * s2 + 64 * 4096 * s2}

    REPEAT = 4      # launches of a kernel per graph: the time of one is the replay's time / REPEAT

    def _build_graphs(self):
        """One CUDA graph per kernel, REPEAT launches each, so that the timed region holds kernels and
        not the host work of an autograd call (which is 2-5x the kernels' own time at these sizes)."""
        t, fn = self.t, self.fn
        grad = torch.autograd.grad
        # autograd runs a backward node on the stream its forward ran on, so the forward passes whose
        # backward is captured run on the capture stream too
        cap = torch.cuda.Stream(device=self.dev)
        cap.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cap):
            yc = fn["conv"](t["x"], t["w"], t["b"], "silu")
            o, z = fn["norm"](t["h"], t["g"], None, residual=t["r"], prenorm=True)
            loss = fn["xent"](t["logits"], t["labels"])
            bodies = [
                lambda: fn["conv"](t["x"], t["w"], t["b"], "silu"),
                lambda: grad(yc, [t["x"], t["w"], t["b"]], t["gconv"], retain_graph=True),
                lambda: fn["norm"](t["h"], t["g"], None, residual=t["r"], prenorm=True),
                lambda: grad([o, z], [t["h"], t["r"], t["g"]], [t["gnorm"], t["gnorm"]], retain_graph=True),
                lambda: fn["xent"](t["logits"], t["labels"]),
                lambda: grad(loss, [t["logits"]], retain_graph=True),
                lambda: fn["lin"](t["xs"], t["wx"]),
            ]
            for body in bodies:                       # warm-up outside capture
                body()
        torch.cuda.current_stream().wait_stream(cap)
        torch.cuda.synchronize()
        self.graphs = []
        for k, body in enumerate(bodies):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cap):
                if k == 6:
                    with torch.no_grad():
                        for _ in range(self.REPEAT):
                            body()
                else:
                    for _ in range(self.REPEAT):
                        body()
            self.graphs.append(g)
        self._loss = loss.detach()

    def step(self, record=False):
        if getattr(self, "graphs", None) is None:
            self._build_graphs()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(8)] if record else None
        for k, g in enumerate(self.graphs):
            if record:
                ev[k].record()
            g.replay()
        if record:
            ev[7].record()
            self.ev.append(ev)
        return self._loss

    def e2e_step(self):
        with torch.no_grad():
            self.t["x"].copy_(self.h_x, non_blocking=True)
        return float(self.step().item())

    def e2e_bytes(self):
        return self.h_x.numel() * 2, 4

    def kernel_rooflines(self):
        names = ("conv1d_fwd", "conv1d_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "xent_fwd", "xent_bwd", "skinny_linear")
        out = {}
        for i, n in enumerate(names):
            out[n] = (self.bytes[n], statistics.mean(e[i].elapsed_time(e[i + 1]) for e in self.ev) / self.REPEAT)
        return out

    cpu_sample = "convolution + norm forward on 1 of 8 sequences (float32, PyTorch ops of the oracle)"

    def cpu_step(self):
        from oracle import scan_oracle as O
        if not hasattr(self, "_cpu"):
            g = torch.Generator().manual_seed(0)
            self._cpu = (torch.randn(1, self.d_inner, self.L, generator=g), torch.randn(self.d_inner, 4, generator=g),
                         torch.randn(self.L, self.d_model, generator=g), torch.ones(self.d_model))
        x, w, h, gw = self._cpu
        O.causal_conv1d_oracle(x, w, None, "silu")
        O.rms_norm_oracle(h, gw, None, 1e-5)
        return self.L


class LmTrain:
    """benchmark configuration 2: Mamba LM, 24 layers, d_model 768 (d_inner 1536, dstate 16, dt_rank 48,
    conv 4), vocabulary 50280, random-init bf16 weights, token ids uniform in [0, 50280), batch 8 x
    2048 tokens, forward + backward of the shifted cross-entropy + a fused AdamW step.  The batch
    is split over the ranks (fixed total work); the gradients are averaged with one flat NCCL
    all-reduce inside the captured step graph (DistributedDataParallel if the capture is refused)."""
    name = "lm_cfg2"
    dtype = "bf16 weights and activations, f32 scan state"
    metric, unit = "training tokens/s (LM forward + backward + optimizer step)", "tokens/s"
    scaling = "strong"
    roofline_note = ("whole training step against the dense bf16 rate: 6 x parameters x tokens floating-point operations "
                     "(projections and LM head); the scan, convolution and norm kernels inside it are HBM / SFU bound")

    def __init__(self, batch=8, L=2048, d_model=768, n_layer=24, vocab=50280):
        self.batch, self.L, self.d_model, self.n_layer, self.vocab = batch, L, d_model, n_layer, vocab
        self.describe = {"workload": f"{self.name}: Mamba LM {n_layer} layers d_model {d_model} vocab {vocab}, "
                                     f"batch {batch} x {L} tokens, fwd + bwd + AdamW",
                         "global_batch": batch, "seq_len": L,
                         "l2": "weights, activations and logits of a step (several GB) exceed the 126 MB L2"}

    def setup(self, dev, pg):
        from lrnnx_b200.lm import MambaLMHeadModel
        self.dev, self.pg = dev, pg
        w = torch.distributed.get_world_size() if pg is not None else 1
        r = torch.distributed.get_rank() if pg is not None else 0
        self.local_batch = max(1, self.batch // w)
        self.tokens = self.local_batch * self.L
        self.describe["parallelism"] = f"data parallel: {self.local_batch} of {self.batch} sequences per GPU" if w > 1 else "single GPU"
        torch.manual_seed(0)
        model = MambaLMHeadModel(self.d_model, self.n_layer, self.vocab, device=dev, dtype=torch.bfloat16)
        self.n_params = sum(p.numel() for p in model.parameters())
        g = torch.Generator().manual_seed(r)
        self.h_ids = torch.randint(0, self.vocab, (self.local_batch, self.L), generator=g).pin_memory()
        self.ids = self.h_ids.to(dev)
        self.ev = []
        self.graph = None
        if pg is not None:
            # With a few sequences per rank the step is bound by the host enqueueing ~2000 kernels, not
            # by the GPU: the whole step (forward, loss, backward, one flat gradient all-reduce over
            # NCCL, AdamW) is captured once and replayed.  If the capture is refused the step falls
            # back to DistributedDataParallel enqueued from the host.
            try:
                self.model = model
                self.opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True, capturable=True)
                self._capture_step(w)
                self.describe["parallelism"] += "; whole step replayed from a CUDA graph, one flat gradient all-reduce (NCCL) inside it"
            except Exception as exc:
                torch.cuda.synchronize()
                self.graph = None
                self.describe["parallelism"] += f"; DistributedDataParallel from the host ({type(exc).__name__} during graph capture)"
                self.model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index])
                self.opt = torch.optim.AdamW(self.model.parameters(), lr=1e-4, fused=True)
        else:
            self.model = model
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=1e-4, fused=True)
        self.launches_per_step = self.n_layer * 8 + 2      # conv, scan, norm forward and backward per layer; the loss (this package's kernels)

    def _fwd_bwd_reduce(self, world):
        from lrnnx_b200.ops.cross_entropy import cross_entropy
        logits = self.model(self.ids)
        loss = cross_entropy(logits.view(-1, self.vocab), self.labels(self.ids).view(-1), ignore_index=-100)
        loss.backward()
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        flat = torch.cat([g.reshape(-1) for g in grads])
        torch.distributed.all_reduce(flat, group=self.pg)
        flat.div_(world)
        torch._foreach_copy_(grads, [t.view_as(g) for t, g in zip(flat.split([g.numel() for g in grads]), grads)])
        return loss

    def _capture_step(self, world):
        dev = self.dev
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                     # warm-up: optimizer state, communicator, allocator
            for _ in range(3):
                self.opt.zero_grad(set_to_none=True)
                self._fwd_bwd_reduce(world)
                self.opt.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        self.opt.zero_grad(set_to_none=True)
        with torch.cuda.graph(graph):
            self._loss = self._fwd_bwd_reduce(world)
            self.opt.step()
        self.graph = graph

    def _train(self, ids):
        from lrnnx_b200.ops.cross_entropy import cross_entropy
        if self.graph is not None:                        # ids is the graph's static input buffer
            self.graph.replay()
            return self._loss
        logits = self.model(ids)
        # next-token loss: the last position has no target (ignored) instead of slicing the logits, which
        # would copy them
        loss = cross_entropy(logits.view(-1, self.vocab), self.labels(ids).view(-1), ignore_index=-100)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return loss

    @staticmethod
    def labels(ids):
        lab = torch.full_like(ids, -100)
        lab[:, :-1] = ids[:, 1:]
        return lab

    def step(self, record=False):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(2)] if record else None
        if record:
            e[0].record()
        loss = self._train(self.ids)
        if record:
            e[1].record()
            self.ev.append(e)
        return loss

    def e2e_step(self):
        self.ids.copy_(self.h_ids, non_blocking=True)
        return float(self._train(self.ids).item())

    def e2e_bytes(self):
        return self.h_ids.numel() * 8, 4

    def kernel_rooflines(self):
        ms = statistics.mean(a[0].elapsed_time(a[1]) for a in self.ev)
        return {"lm_train_step": (0, ms, {"tensor_flops": 6.0 * self.n_params * self.tokens})}

    cpu_sample = "2 of 24 layers, 1 sequence of 256 tokens, float32 (extrapolated by layers x tokens)"

    def cpu_step(self):
        from oracle import scan_oracle as O
        if not hasattr(self, "_cpu"):
            from lrnnx_b200.lm import MambaLMHeadModel
            torch.manual_seed(0)
            m = MambaLMHeadModel(self.d_model, 2, self.vocab)
            self._cpu = ({k: v.detach().requires_grad_(True) for k, v in m.state_dict().items()},
                         torch.randint(0, self.vocab, (1, 256)))
        sd, ids = self._cpu
        logits = O.mamba_lm_oracle(sd, ids, 2)
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, self.vocab), ids[:, 1:].reshape(-1))
        torch.autograd.grad(loss, [v for k, v in sd.items() if k != "lm_head.weight"], allow_unused=True)
        return 256 * 2 / self.n_layer


class LmDecode:
    """benchmark configuration 4: Mamba LM at the 1.4B shape (48 layers, d_model 2048, d_inner 4096,
    dstate 16, dt_rank 128), random-init bf16 weights, batch 64 (split over the ranks), random
    prompts of 512 tokens prefilled through the scan kernels, then 256 greedy tokens replayed from
    one captured CUDA graph of the decoding step.  A step of this workload is one whole generation."""
    name = "decode_cfg4"
    dtype = "bf16 weights and activations, f32 scan state"
    metric, unit = "generated tokens/s (prefill 512 + 256 new tokens, CUDA-graph decoding)", "tokens/s"
    scaling = "strong"
    roofline_note = ("decoding is bound by reading the weights (2.7 GB) and the recurrent states (1.7 GB, read and "
                     "written) once per generated token; the fraction is of the measured HBM copy rate")

    def __init__(self, batch=64, prompt=512, new=256, d_model=2048, n_layer=48, vocab=50280):
        self.batch, self.prompt, self.new = batch, prompt, new
        self.d_model, self.n_layer, self.vocab = d_model, n_layer, vocab
        self.describe = {"workload": f"{self.name}: Mamba LM {n_layer} layers d_model {d_model}, batch {batch}, "
                                     f"prompt {prompt}, {new} generated tokens, CUDA-graph replay",
                         "global_batch": batch, "seq_len": prompt + new,
                         "l2": "weights and states read per token (4.4 GB) exceed the 126 MB L2"}

    def setup(self, dev, pg):
        from lrnnx_b200.lm import MambaLMHeadModel
        self.dev, self.pg = dev, pg
        w = torch.distributed.get_world_size() if pg is not None else 1
        r = torch.distributed.get_rank() if pg is not None else 0
        self.local_batch = max(1, self.batch // w)
        self.tokens = self.local_batch * self.new
        self.describe["parallelism"] = f"batch shards: {self.local_batch} of {self.batch} sequences per GPU" if w > 1 else "single GPU"
        torch.manual_seed(0)
        self.model = MambaLMHeadModel(self.d_model, self.n_layer, self.vocab, device=dev, dtype=torch.bfloat16).eval()
        self.n_params = sum(p.numel() for p in self.model.parameters())
        g = torch.Generator().manual_seed(r)
        self.h_prompt = torch.randint(0, self.vocab, (self.local_batch, self.prompt), generator=g).pin_memory()
        self.d_prompt = self.h_prompt.to(dev)
        self.t = []
        self.launches_per_step = self.n_layer * 3 * (self.new - 1) + self.n_layer * 3   # norm, conv update, state update per layer and token; prefill

    def step(self, record=False):
        tm = {} if record else None
        out = self.model.generate(self.d_prompt, self.new, use_cuda_graph=True, timings=tm)
        if record:
            self.t.append(tm)
        return out

    def e2e_step(self):
        self.d_prompt.copy_(self.h_prompt, non_blocking=True)
        return int(self.step().cpu()[0, -1])

    def e2e_bytes(self):
        return self.h_prompt.numel() * 8, self.local_batch * self.new * 8

    def kernel_rooflines(self):
        dec = statistics.mean(t["decode_ms"] for t in self.t) / (self.new - 1)
        pre = statistics.mean(t["prefill_ms"] for t in self.t)
        d_inner = 2 * self.d_model
        state_bytes = self.n_layer * self.local_batch * d_inner * (2 * 16 * 4 + 2 * 4 * 2)     # scan state r+w, conv state r+w
        per_token = 2 * self.n_params + state_bytes
        self.describe["prefill_ms"] = pre
        return {"decode_step_graph": (per_token, dec)}

    cpu_sample = "2 of 48 layers, full batch, one decoding step, float32 (extrapolated by layers)"

    def cpu_step(self):
        from oracle import scan_oracle as O
        if not hasattr(self, "_cpu"):
            from lrnnx_b200.lm import MambaLMHeadModel
            torch.manual_seed(0)
            m = MambaLMHeadModel(self.d_model, 2, self.vocab)
            sd = {k: v.detach() for k, v in m.state_dict().items()}
            d_inner = 2 * self.d_model
            states = [(torch.zeros(self.batch, d_inner, 4), torch.zeros(self.batch, d_inner, 16)) for _ in range(2)]
            self._cpu = (sd, states, torch.randint(0, self.vocab, (self.batch,)))
        sd, states, tok = self._cpu
        with torch.no_grad():
            O.mamba_lm_step_oracle(sd, tok, states, 2)
        return self.batch * 2 / self.n_layer


def make_workload(name, sub=False):
    """``sub``: the workload is a sub-record of the default run (bounded CPU sample)."""
    if name in ("s5_scan", "s5_scan_cfg1", "default"):
        return S5Scan(cpu_full=not sub)
    if name == "s5_scan_zoh":
        return S5Scan(disc="zoh", name="s5_scan_zoh", cpu_full=False)
    if name == "s5_strong":
        return S5Scan(name="s5_strong_cfg1", strong=True, cpu_full=False)
    if name == "s6_cfg0":
        return S6Scan("s6_cfg0", 2, 256, 512, 16, torch.float32)
    if name == "s6_layer":
        return S6Scan("s6_layer_cfg2", 8, 1536, 2048, 16, torch.bfloat16)
    if name == "s6_layer_f32":
        return S6Scan("s6_layer_f32", 8, 1536, 2048, 16, torch.float32)
    if name == "s6_long":
        return S6Scan("s6_long_cfg3", 1, 5120, 131072, 16, torch.bfloat16, backward=False)
    if name in ("ssu_step", "ssu_step_cfg4"):
        return SsuStep()
    if name in ("cauchy", "cauchy_s4"):
        return CauchyKernel()
    if name in ("block_kernels", "block_kernels_cfg2"):
        return BlockKernels()
    if name == "lm_cfg2":
        return LmTrain()
    if name == "decode_cfg4":
        return LmDecode()
    raise SystemExit(f"unknown workload {name}")


SUB_WORKLOADS = ("s6_cfg0", "s6_layer", "s6_layer_f32", "s6_long", "ssu_step", "cauchy", "s5_scan_zoh", "block_kernels",
                 "lm_cfg2", "decode_cfg4")

# nominal fp32 rate of one B200: 148 SMs x 128 FMA lanes x 2 x 1.965 GHz (no measured figure exists)
FP32_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


# --------------------------------------------------------------------------- arms
def time_cpu(wl, steps, warmup):
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(warmup):
        wl.cpu_step()
    t0 = time.perf_counter()
    toks = 0.0
    for _ in range(steps):
        toks += wl.cpu_step()
    dt = time.perf_counter() - t0
    return toks / dt, dt / steps


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = min(args.steps, 3), min(args.warmup, 1)
    tps, sec = time_cpu(wl, steps, warmup)
    line = {"impl": "reference", "metric": wl.metric, "value": tps, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded)", "config": wl.describe,
            "cpu_baseline": {"value": tps, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": wl.cpu_sample},
            "e2e": {"value": tps, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(json.dumps(line))


def measure(wl, steps, warmup, world, rank, local, dev, pg, sample_clocks=True):
    """Set up one workload and time it; returns its record on rank 0 (None on the other ranks)."""
    wl.setup(dev, pg)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(fn, n, w, record=False, flush=None):
        """n steps between two barriers.  Workloads whose operands fit in the L2 get a 256 MB write
        before every step; the time of a step is then taken between events that bracket the step
        alone (the flush writes are not part of the workload), and the steps' times are summed."""
        for _ in range(w):
            if flush is not None:
                flush.zero_()
            fn()
        barrier()
        drain = getattr(wl, "drain", None)
        if flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn(record=True) if record else fn()
            if drain is not None:
                drain()          # the current stream waits for collectives still in flight on NCCL's stream
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
        else:
            pairs = []
            for i in range(n):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn(record=True) if record else fn()
                if drain is not None and i == n - 1:
                    drain()
                b.record()
                pairs.append((a, b))
            barrier()
            ms = sum(a.elapsed_time(b) for a, b in pairs)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n

    sampler = ClockSampler(local) if (rank == 0 and sample_clocks) else None
    if sampler:
        sampler.start()
    ms_step = timed(wl.step, steps, warmup, record=True, flush=getattr(wl, "flush_buf", None))
    clocks = sampler.stop() if sampler else None
    e2e_steps = max(3, min(steps, 10))
    ms_e2e = timed(wl.e2e_step, e2e_steps, 3)
    check = wl.sp_check() if getattr(wl, "sp", False) else None
    if rank != 0:
        return None

    peak, peak_kind = measured_peaks()
    roofs = {}
    for kname, item in wl.kernel_rooflines().items():
        nbytes, ms = item[0], item[1]
        extra = item[2] if len(item) > 2 else {}
        ach = nbytes / (ms * 1e-3) / 1e9
        roofs[kname] = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                        "traffic": NCU_TRAFFIC.get((wl.name, kname)), "algorithmic_bytes": nbytes,
                        "ms_per_launch": ms, "peak_source": peak_kind}
        if "tensor_flops" in extra:     # a step bound by dense bf16 GEMMs: fraction of the measured (sustained) rate
            tf = extra["tensor_flops"] / (ms * 1e-3) / 1e12
            tpeak, tkind = measured_tensor_peak()
            roofs[kname] = {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                            "traffic": None, "algorithmic_flops": extra["tensor_flops"], "ms_per_launch": ms,
                            "peak_source": tkind}
        if "flops" in extra:     # a kernel bound by the fp32 pipe: the fraction is of the fp32 rate
            tf = extra["flops"] / (ms * 1e-3) / 1e12
            roofs[kname].update({"bound": "fp32", "achieved": tf, "peak": FP32_PEAK_TFLOPS, "unit": "TFLOP/s",
                                 "frac": tf / FP32_PEAK_TFLOPS, "algorithmic_flops": extra["flops"],
                                 "peak_source": "nominal: 148 SMs x 128 lanes x 2 x 1.965 GHz", "hbm_frac": ach / peak})
        note = getattr(wl, "roofline_note", None)
        if note:
            roofs[kname]["note"] = note
    dominant = max(roofs, key=lambda k: roofs[k]["ms_per_launch"])
    # the CPU baseline is taken at N = 1 only (the other ranks would wait for rank 0's host work)
    cpu_tps, cpu_sec = time_cpu(wl, 1, 0) if world == 1 else (None, None)
    h2d, d2h = wl.e2e_bytes()
    strong = getattr(wl, "scaling", "weak") == "strong"
    total_tokens = wl.tokens * (1 if (strong and getattr(wl, "sp", False)) else world)
    describe = dict(wl.describe)
    if "global_batch" in describe and not strong:
        describe["global_batch"] = describe["global_batch"] * world     # weak scaling: every rank runs its own full batch
    rec = {"metric": wl.metric, "value": total_tokens / (ms_step * 1e-3), "unit": wl.unit,
           "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
           "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
           "dtype": wl.dtype,
           "data": "synthetic (seeded CPU generator, copied to the GPU)", "config": describe,
           "clocks": clocks,
           "e2e": {"value": total_tokens / (ms_e2e * 1e-3), "unit": wl.unit, "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
           "gpu_launches": wl.launches_per_step * steps,
           "roofline": dict(roofs[dominant], kernel=dominant),
           "kernels": roofs,
           "cpu_baseline": {"value": cpu_tps, "unit": wl.unit, "cores": torch.get_num_threads(),
                            "kind": "port", "sample": wl.cpu_sample if world == 1 else "not timed at N > 1",
                            "seconds": cpu_sec}}
    if check is not None:
        rec["sp_check"] = check
    return rec


def run_ours(args, wl, with_subs):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    pg = None
    if world > 1:
        # a rank that lost its peers must not sit in a collective for ever: leave after 20 minutes
        # (a healthy multi-rank run of every workload takes one to two)
        import threading
        guard = threading.Timer(1200.0, lambda: (sys.stderr.write("bench.py: multi-rank run exceeded 20 minutes, leaving\n"),
                                                 os._exit(3)))
        guard.daemon = True
        guard.start()
        torch.distributed.init_process_group("nccl", device_id=dev)
        pg = torch.distributed.group.WORLD
    line = measure(wl, args.steps, args.warmup, world, rank, local, dev, pg)
    failed = False
    if with_subs:
        subs = {}
        names = SUB_WORKLOADS + (("s5_strong",) if world > 1 else ())
        del wl
        for name in names:
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            sub = make_workload(name, sub=True)
            rec = measure(sub, max(3, min(args.steps, 10)), 3, world, rank, local, dev, pg, sample_clocks=True)
            if rec is not None:
                # a sub-record keeps what differs from the top-level line
                for k in ("higher_is_better", "vs_baseline", "data", "n_gpus"):
                    rec.pop(k, None)
                subs[name] = rec
                if rec.get("sp_check") is not None and not rec["sp_check"]["ok"]:
                    failed = True
            del sub
        if rank == 0:
            line["workloads"] = subs
    elif rank == 0 and line.get("sp_check") is not None and not line["sp_check"]["ok"]:
        failed = True
    if world > 1:
        flag = torch.tensor([1 if failed else 0], device=dev)
        torch.distributed.broadcast(flag, 0)
        failed = bool(flag.item())
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.cuda.synchronize()
    if rank == 0:
        emit(json.dumps(line))
    if failed:
        sys.stderr.write("bench.py: the sequence-parallel output differs from the unsplit forward (sp_check)\n")
    if world > 1:
        # Leave without running destructors: tearing down a communicator whose collectives were
        # captured in CUDA graphs can block for minutes in the communicator's destroy call, after
        # every number has been produced.  All ranks have passed the barrier above.
        sys.stderr.flush()
        os._exit(1 if failed else 0)
    if failed:
        raise SystemExit(1)


_JSON_FD = None


def emit(text):
    """Write the result line to the process's original stdout."""
    if _JSON_FD is None:
        print(text, flush=True)
    else:
        os.write(_JSON_FD, (text + "\n").encode())


def main():
    # Libraries (the collective library prints its version banner) write to file descriptor 1;
    # the result line must be the only thing on stdout, so everything else is sent to stderr.
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, help="run one workload alone (default: configs[1] plus the sub-records)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = make_workload(args.workload or "s5_scan_cfg1")
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl, with_subs=args.workload is None)


if __name__ == "__main__":
    main()
