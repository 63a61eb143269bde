#!/usr/bin/env python
"""Benchmark of the KDA recurrent core on B200: batched single-token decode (state GB/s against the HBM roofline).

One step = the decode of one token for every slot across all 34 KDA layers of the model: 34 launches of
glm53f_kda_core_decode_batch, one per layer, each over 16 slots x 64 heads with its own bf16 state
(16 x 2 MiB read + 16 x 2 MiB written per layer).  The 34 layers' states are distinct buffers (1.06 GiB in all),
so every launch streams its states from HBM: the working set is ~8x the 126 MB L2.

  value     state GB/s with the token inputs already resident in HBM (CUDA events around K steps)
  e2e       the same metric through the host-facing API: each step copies its token inputs from pinned host memory,
            runs the 34 launches and reads the 34 layers' outputs back
  roofline  algorithmic state bytes per launch / mean launch time, against the measured HBM copy bandwidth
  cpu_baseline   the CPU oracle (the reference's recurrence restated in C++) on all host cores, on a bounded sample

`--impl reference` times the reference instead and prints the same line with "impl": "reference": the reference's
OWN CUDA kernels (compiled from the reference tree by `make -C oracle ref` into oracle/_ref, unmodified, for sm_100a)
on the same GPU, same shapes, same CUDA-graph and event timing, entered through the reference's own symbol for this
step (glm53f_kda_chain_batch_bf16state); its CPU formulation (the oracle port: the reference's CPU code is Rust and
no Rust toolchain exists on this machine) is the line's `cpu_baseline`, and the whole arm when oracle/_ref is absent.
With torchrun (N > 1) every rank decodes its own 16 slots (slots are independent units: no collective on the data
path); the time is the maximum over ranks and `value` the whole job's.
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADS, LAYERS, SLOTS, DK = 64, 34, 16, 128
STATE_ELEMS = HEADS * DK * DK                        # one slot, one layer
STATE_BYTES_PER_LAUNCH = 2 * SLOTS * STATE_ELEMS * 2  # bf16 read + write = 64 MiB
TOKEN_IN_BYTES = HEADS * DK * (2 + 2 + 2 + 4) + HEADS * 4  # q, k, v bf16 + g f32 + beta f32 per token
TOKEN_OUT_BYTES = HEADS * DK * 2
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the decode kernel: the mean over 16 consecutive launches
# of an 8-layer step (256 MiB of distinct states, caches left as they are between launches, so that one launch's
# writes are evicted during the next ones as in the timed run); summarised under profiles/.
NCU_DRAM_BYTES_PER_LAUNCH = 34_876_112 + 32_331_792
# The same for the prefill kernel: 601 MB per captured launch of 2,048 (chain, chunk) items = 32 chunks of all 64 heads.
NCU_PREFILL_DRAM_BYTES_PER_TOKEN = (393_953_280 + 207_395_072) // (32 * 64)


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons.  nvidia-smi needs a fraction of a second to start and samples
    every 20 ms at best, while a timed region of 20 decode steps lasts 11 ms, so the sampler is started early, every
    sample carries its timestamp, and the caller names the window to evaluate: the timed region followed by a short
    untimed tail in which the same CUDA graph keeps replaying (the same load, so the same clocks)."""

    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self, t0=None, t1=None, t_timed_end=None):
        """Samples taken in [t0, t1] (epoch seconds; all samples when None); `t_timed_end` splits the timed region from the tail."""
        import datetime

        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons, in_timed = [], [], set(), 0
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clock, cmax = float(f[2]), float(f[3])
            except ValueError:
                continue
            if t0 is not None and not (t0 - 0.02 <= ts <= t1 + 0.02):
                continue
            sm.append(clock)
            mx.append(cmax)
            if t_timed_end is not None and ts <= t_timed_end + 0.02:
                in_timed += 1
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[6:10]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_in_timed_region": in_timed,
                "window": "the timed region and 0.4 s of the same graph replaying after it"}


def oracle_module():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import kda_oracle

    kda_oracle.build()
    return kda_oracle


# ---- the layer ABI (the thirteen drop-in symbols) on the engine's argument values --------------------------------------
P_STRIDE, B_OFF, AG_STRIDE, OUT_STRIDE, CONV_CH = 24_640, 24_576, 16_384, 8_192, 3 * HEADS * DK  # crates/glm53f-forward/src/shape.rs:22-32
LAYER_IN_BYTES = (P_STRIDE + AG_STRIDE) * 2   # one token's projection row and gate rows
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libglm53f_kda_ref.so")


def reference_library(pkg):
    """The reference's own kernels (oracle/_ref, built from the reference tree), typed like the product's; None when absent."""
    if not os.path.exists(REF_LIB):
        return None
    lib = C.CDLL(REF_LIB)
    for name in pkg.ffi.REFERENCE_SYMBOLS:
        res, argtypes = pkg.ffi.SIGNATURES[name]
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, argtypes
    return lib


class LayerAbi:
    """Inputs of the layer entry points with the forward's argument values (p rows [q|k|v|b] of 24,640, beta logits at
    24,576, the interleaved [a|g] gate rows of 16,384, out rows of 8,192, eps 1e-5, lower -5; slot-major state and conv
    arenas per layer), and the three steps of the engine through them, for any library exporting the thirteen symbols."""

    def __init__(self, torch, rank, slots, rows_per_slot, layers, bf16_state=True, seed=0):
        self.torch, self.slots, self.rps, self.layers, self.bf16 = torch, slots, rows_per_slot, layers, bf16_state
        gen = torch.Generator(device="cuda").manual_seed(0x53454544 + 31 + 97 * rank + seed)
        rows = self.rows = slots * rows_per_slot
        rn = lambda n, s=1.0: (torch.randn(n, device="cuda", generator=gen) * s)
        self.p = rn(layers * rows * P_STRIDE).to(torch.bfloat16)
        self.ag = rn(layers * rows * AG_STRIDE).to(torch.bfloat16)
        self.conv = rn(layers * slots * 3 * CONV_CH).to(torch.bfloat16)
        self.conv_w = rn(CONV_CH * 4, 0.5).to(torch.bfloat16)
        self.a_log, self.dt_bias = rn(HEADS, 0.5), rn(HEADS * DK)
        self.norm_w = (1.0 + rn(DK, 0.1)).to(torch.bfloat16)
        st = rn(layers * slots * STATE_ELEMS, 0.05)
        self.state = st.to(torch.bfloat16) if bf16_state else st
        self.out = torch.empty(layers * rows * OUT_STRIDE, dtype=torch.bfloat16, device="cuda")
        self.cu = torch.arange(slots + 1, dtype=torch.int32, device="cuda") * rows_per_slot
        self.conv_off = torch.arange(slots, dtype=torch.int64, device="cuda") * (3 * CONV_CH)
        self.state_off = torch.arange(slots, dtype=torch.int64, device="cuda") * STATE_ELEMS

    def at(self, t, elems):
        return C.c_void_p(t.data_ptr() + elems * t.element_size())

    def chain(self, lib, l, stream, write_state=True, saves=None, p=None, ag=None, out=None):
        """One layer's chain over every slot's rows (decode: one row each; verify: the window, states untouched)."""
        r, P = self.rows, lambda t: C.c_void_p(t.data_ptr())
        p_at = self.at(self.p, l * r * P_STRIDE) if p is None else p
        ag_t, ag_e = (self.ag, l * r * AG_STRIDE) if ag is None else ag
        st = self.at(self.state, l * self.slots * STATE_ELEMS)
        fn = lib.glm53f_kda_chain_batch_bf16state if self.bf16 else lib.glm53f_kda_chain_batch
        sv = [None] * 4 if saves is None else saves
        rc = fn(HEADS, self.slots, P(self.cu), p_at, P_STRIDE, B_OFF, self.at(ag_t, ag_e), AG_STRIDE, self.at(ag_t, ag_e + 8192), AG_STRIDE,
                self.at(self.conv, l * self.slots * 3 * CONV_CH), P(self.conv_off), P(self.conv_w), st, st if write_state else None,
                P(self.state_off), P(self.a_log), P(self.dt_bias), P(self.norm_w), 1e-5, -5.0,
                self.at(self.out, l * r * OUT_STRIDE) if out is None else out, OUT_STRIDE, *sv, stream)
        if rc != 0:
            raise RuntimeError(f"chain launch failed: {rc}")

    def prefill(self, lib, l, stream, ws, ws_bytes, max_rows, value_blocks=0):
        r, P = self.rows, lambda t: C.c_void_p(t.data_ptr())
        st = self.at(self.state, l * self.slots * STATE_ELEMS)
        fn = lib.glm53f_kda_prefill_batch_bf16state if self.bf16 else lib.glm53f_kda_prefill_batch
        rc = fn(HEADS, self.slots, P(self.cu), max_rows, self.at(self.p, l * r * P_STRIDE), P_STRIDE, B_OFF,
                self.at(self.ag, l * r * AG_STRIDE), AG_STRIDE, self.at(self.ag, l * r * AG_STRIDE + 8192), AG_STRIDE,
                self.at(self.conv, l * self.slots * 3 * CONV_CH), P(self.conv_off), P(self.conv_w), st, st, P(self.state_off),
                P(self.a_log), P(self.dt_bias), P(self.norm_w), 1e-5, -5.0, self.at(self.out, l * r * OUT_STRIDE), OUT_STRIDE,
                value_blocks, P(ws), ws_bytes, stream)
        if rc != 0:
            raise RuntimeError(f"prefill launch failed: {rc}")


def graph_ms(torch, fn, reps, warm=3):
    """`fn(stream)` captured once in a CUDA graph on a side stream, replayed `reps` times between events."""
    torch.cuda.synchronize()  # the inputs (metadata arrays included) were written on the current stream
    side = torch.cuda.Stream()
    st = C.c_void_p(side.cuda_stream)
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn(st)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fn(st)
    torch.cuda.synchronize()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, graph


def run_layer_abi(torch, lib, rank, layers, steps, prefill_lib_ok=True):
    """The engine's three steps through the drop-in symbols of `lib` (the product, or the reference's own kernels):
    decode (config 1's shape: 16 slots x 1 row x `layers` layers, bf16 states), verify + commit (config 4's shape:
    48 slots x 16 rows, saves written, states untouched, then glm53f_kda_replay_batch_bf16state over every layer)
    and the prefill lanes (config 2's engine shape: 4 lanes x 2,048 rows, glm53f_kda_prefill_batch[_bf16state])."""
    import numpy as np

    hbm, kind = peaks()
    res = {"arguments": {"p_stride": P_STRIDE, "b_off": B_OFF, "ag_stride": AG_STRIDE, "out_stride": OUT_STRIDE, "eps": 1e-5, "lower": -5.0}}
    # decode
    d = LayerAbi(torch, rank, SLOTS, 1, layers)
    ms, _g = graph_ms(torch, lambda st: [d.chain(lib, l, st) for l in range(layers)], steps)
    gbs = layers * STATE_BYTES_PER_LAUNCH / (ms * 1e-3) / 1e9
    res["decode"] = {"entry": "glm53f_kda_chain_batch_bf16state", "ms_per_step": ms, "state_gbs": gbs, "frac_of_hbm": gbs / hbm, "gpu_launches": layers}
    del d, _g
    torch.cuda.empty_cache()
    # verify + commit
    v = LayerAbi(torch, rank, VERIFY_SLOTS, VERIFY_WINDOW, layers)
    nkv, nb = v.rows * HEADS * DK, v.rows * HEADS
    ks, gs_ = torch.empty(layers * nkv, device="cuda"), torch.empty(layers * nkv, device="cuda")
    vs, bs = torch.empty(layers * nkv, dtype=torch.bfloat16, device="cuda"), torch.empty(layers * nb, device="cuda")
    keep = torch.tensor(np.random.default_rng(0x53454548).integers(0, VERIFY_WINDOW + 1, VERIFY_SLOTS), dtype=torch.int32, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())

    def verify(st):
        for l in range(layers):
            v.chain(lib, l, st, write_state=False, saves=[v.at(ks, l * nkv), v.at(vs, l * nkv), v.at(gs_, l * nkv), v.at(bs, l * nb)])

    def commit(st):
        rc = lib.glm53f_kda_replay_batch_bf16state(HEADS, layers, VERIFY_SLOTS, P(v.cu), P(keep), P(v.state), P(v.state), VERIFY_SLOTS * STATE_ELEMS,
                                                   P(v.state_off), P(ks), P(vs), P(gs_), P(bs), nkv, nb, st)
        if rc != 0:
            raise RuntimeError(f"replay launch failed: {rc}")

    n = max(2, steps // 5)
    ms_v, _g1 = graph_ms(torch, verify, n, warm=2)
    ms_c, _g2 = graph_ms(torch, commit, n, warm=2)
    sb = layers * VERIFY_SLOTS * STATE_ELEMS * 2
    res["verify"] = {"entry": "glm53f_kda_chain_batch_bf16state (state_out NULL, saves)", "ms_per_step": ms_v, "rows_per_s": v.rows * layers / (ms_v * 1e-3),
                     "state_gbs": sb / (ms_v * 1e-3) / 1e9, "frac_of_hbm": sb / (ms_v * 1e-3) / 1e9 / hbm}
    res["commit"] = {"entry": "glm53f_kda_replay_batch_bf16state", "ms_per_step": ms_c, "state_gbs": 2 * sb / (ms_c * 1e-3) / 1e9,
                     "frac_of_hbm": 2 * sb / (ms_c * 1e-3) / 1e9 / hbm}
    if hasattr(lib, "glm53f_kda_verify_mode"):  # the product's tensor-core form of the same call (two launches a layer)
        set_v = lib.glm53f_kda_verify_mode
        set_v.restype, set_v.argtypes = C.c_int32, [C.c_int32]
        set_v(1)
        try:
            ms_t, _g3 = graph_ms(torch, verify, n, warm=2)
        finally:
            set_v(0)
        # all the bytes the step must move: states read once, projection rows, gate rows in; outputs and saves out
        vb = sb + layers * v.rows * ((P_STRIDE + AG_STRIDE) * 2 + OUT_STRIDE * 2 + HEADS * 1284)
        res["verify_chunked"] = {"entry": "glm53f_kda_chain_batch_bf16state after glm53f_kda_verify_mode(1)", "ms_per_step": ms_t,
                                 "rows_per_s": v.rows * layers / (ms_t * 1e-3), "state_gbs": sb / (ms_t * 1e-3) / 1e9, "gpu_launches": 2 * layers,
                                 "algorithmic_bytes": vb,
                                 "roofline": {"bound": "hbm", "achieved": vb / (ms_t * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                                              "frac": vb / (ms_t * 1e-3) / 1e9 / hbm, "peak_source": kind}}
        del _g3
    del v, ks, gs_, vs, bs, _g1, _g2
    torch.cuda.empty_cache()
    # prefill lanes: 4 lanes x 2,048 rows in one call, and one lane per call; f32 and bf16 states
    lanes, lane_rows, pl = 4, 2048, min(layers, 2)
    res["prefill_layer"] = {"workload": f"{lanes} lanes x {lane_rows} rows, 64 heads, through glm53f_kda_prefill_batch[_bf16state]; ms per lane and layer",
                            "reference_published_ms_per_lane": {"value": 0.983, "where": "RTX 5090, docs/PERFORMANCE.md:374-378"}}
    try:
        set_mode = lib.glm53f_kda_prefill_mode
        set_mode.restype, set_mode.argtypes = C.c_int32, [C.c_int32]
        modes = [("exact", 0), ("chunked", 1)]   # the product: the row-by-row form (default) and the tensor-core form
    except AttributeError:
        set_mode, modes = None, [("kernel", None)]  # the reference's kernels have one form
    for mode_name, mode in modes:
        if set_mode is not None:
            set_mode(mode)
        try:
            for bf16 in (False, True):
                for batch in (lanes, 1):
                    f = LayerAbi(torch, rank, batch, lane_rows, pl, bf16_state=bf16, seed=5)
                    wsb = int(lib.glm53f_kda_prefill_workspace_bytes(HEADS, batch, 256))
                    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device="cuda")
                    try:
                        ms, _g = graph_ms(torch, lambda st: [f.prefill(lib, l, st, ws, wsb, lane_rows, 2) for l in range(pl)], max(2, steps // 5), warm=2)
                        res["prefill_layer"][f"{mode_name}_" + ("bf16state" if bf16 else "f32state") + f"_batch{batch}"] = {
                            "ms_per_lane": ms / pl / batch, "rows_per_s": batch * lane_rows * pl / (ms * 1e-3), "workspace_bytes": wsb,
                            "rows_per_pass": 256, "value_blocks": 2}
                        del _g
                        if mode == 1 and batch == lanes and not bf16:
                            # the same call with a workspace for a whole lane per pass (the reference's default is 256 rows)
                            wsb2 = int(lib.glm53f_kda_prefill_workspace_bytes(HEADS, batch, lane_rows))
                            ws2 = torch.empty(wsb2, dtype=torch.uint8, device="cuda")
                            ms2, _g = graph_ms(torch, lambda st: [f.prefill(lib, l, st, ws2, wsb2, lane_rows, 2) for l in range(pl)], max(2, steps // 5), warm=2)
                            res["prefill_layer"][f"{mode_name}_f32state_batch{batch}_whole_lane_passes"] = {
                                "ms_per_lane": ms2 / pl / batch, "rows_per_s": batch * lane_rows * pl / (ms2 * 1e-3), "workspace_bytes": wsb2,
                                "rows_per_pass": lane_rows, "value_blocks": 2}
                            del _g, ws2
                    finally:
                        del f, ws
                        torch.cuda.empty_cache()
        finally:
            if set_mode is not None:
                set_mode(0)
    return res


def cpu_decode_gbs(seconds: float, layers_sample: int = 2):
    """The CPU oracle's decode (kernel-order recurrence, bf16-rounded states) on every host core: state GB/s counted
    as for the GPU (2 bytes read + 2 written per state element)."""
    import numpy as np

    o = oracle_module()
    pkg = importlib.import_module("glm53f-afd_b200")
    cores = os.cpu_count() or 1
    toks = [pkg.synth.tokens(1, l, SLOTS, HEADS) for l in range(layers_sample)]
    rng = np.random.default_rng(1)
    states = [o.bf16_round_np((rng.standard_normal(SLOTS * STATE_ELEMS) * 0.05).astype(np.float32)) for _ in range(layers_sample)]
    cu = np.arange(SLOTS + 1, dtype=np.int32)
    offs = np.arange(SLOTS, dtype=np.int64) * STATE_ELEMS
    lib = o.lib()
    f32p, u16p = C.POINTER(C.c_float), C.POINTER(C.c_uint16)
    args = []
    for l in range(layers_sample):
        q, k, v, g, b = toks[l]
        y = np.zeros(SLOTS * HEADS * DK, np.float32)
        args.append((q, k, v, g, b, states[l], y))
    steps, t0 = 0, time.perf_counter()
    while True:
        for q, k, v, g, b, s, y in args:
            lib.kdao_core_step_batch(C.c_int(HEADS), C.c_int(SLOTS), cu.ctypes.data_as(C.POINTER(C.c_int32)),
                                     q.ctypes.data_as(u16p), k.ctypes.data_as(u16p), v.ctypes.data_as(u16p),
                                     g.ctypes.data_as(f32p), b.ctypes.data_as(f32p), s.ctypes.data_as(f32p),
                                     offs.ctypes.data_as(C.POINTER(C.c_int64)), C.c_int(1), C.c_int(0), C.c_int(cores),
                                     y.ctypes.data_as(f32p), None, None, None, None)
        steps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    gbs = steps * layers_sample * STATE_BYTES_PER_LAUNCH / dt / 1e9
    return gbs, cores, f"{steps} steps x {layers_sample} of 34 layers x {SLOTS} slots x {HEADS} heads in {dt:.1f} s"


VERIFY_SLOTS, VERIFY_WINDOW = 48, 16  # config 4: draft verification and rollback over all layers


def run_verify(torch, lib, rank, layers, steps):
    """Config 4: per step, every layer verifies 16 draft rows for each of 48 slots (states read, not written; replay
    inputs saved), then one commit over all layers rolls every slot's state forward to its accepted prefix (drawn from
    0..16).  Algorithmic bytes: verify reads each bf16 state once; the commit reads and writes it once."""
    import ctypes as C

    import numpy as np

    slots, window = VERIFY_SLOTS, VERIFY_WINDOW
    rows, per = slots * window, STATE_ELEMS
    gen = torch.Generator(device="cuda").manual_seed(0x53454544 + 4 + 97 * rank)
    n = rows * HEADS

    def unit(scale):
        x = torch.randn(n, DK, device="cuda", generator=gen)
        return (x * (scale / torch.sqrt((x * x).sum(1, keepdim=True) + 1e-6))).to(torch.bfloat16).reshape(-1)

    # one set of draft inputs serves every layer (the timing does not depend on the values); states are per layer
    q, k = unit(DK ** -0.5), unit(1.0)
    v = torch.randn(n * DK, device="cuda", generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(n * DK, device="cuda", generator=gen) + 3.0)
    beta = torch.sigmoid(torch.randn(n, device="cuda", generator=gen))
    arena = (torch.randn(layers * slots * per, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    keeps = np.random.default_rng(0x53454548).integers(0, window + 1, slots)
    cu = torch.arange(slots + 1, dtype=torch.int32, device="cuda") * window
    keep = torch.tensor(keeps, dtype=torch.int32, device="cuda")
    off = torch.arange(slots, dtype=torch.int64, device="cuda") * per
    nkv, nb = rows * HEADS * DK, rows * HEADS
    ks, gs_ = torch.empty(layers * nkv, device="cuda"), torch.empty(layers * nkv, device="cuda")
    vs = torch.empty(layers * nkv, dtype=torch.bfloat16, device="cuda")
    bs = torch.empty(layers * nb, device="cuda")
    out = torch.empty(rows * HEADS * DK, dtype=torch.bfloat16, device="cuda")
    P = lambda t, byte_off=0: C.c_void_p(t.data_ptr() + byte_off)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def verify(flags=0):
        for l in range(layers):
            rc = lib.glm53f_kda_core_verify_batch(HEADS, slots, P(cu), P(q), P(k), P(v), P(g), P(beta), P(arena, 2 * l * slots * per), None, P(off),
                                                  1, flags, None, None, 1e-5, P(out), P(ks, 4 * l * nkv), P(vs, 2 * l * nkv), P(gs_, 4 * l * nkv),
                                                  P(bs, 4 * l * nb), stream)
            if rc != 0:
                raise RuntimeError(f"verify launch failed: {rc}")

    def verify_tensor():
        verify(2)  # GLM53F_KDA_CORE_TENSOR: the window as one 16-row chunk on the tensor cores

    def commit():
        rc = lib.glm53f_kda_core_commit_batch(HEADS, layers, slots, P(cu), P(keep), P(arena), P(arena), slots * per, P(off), 1, P(ks), P(vs),
                                              P(gs_), P(bs), nkv, nb, stream)
        if rc != 0:
            raise RuntimeError(f"commit launch failed: {rc}")

    def timed(fn):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for _ in range(3):
        verify()
        commit()
    verify_tensor()
    ms_v, ms_c, ms_t = timed(verify), timed(commit), timed(verify_tensor)
    ms_ct = None
    if hasattr(lib, "glm53f_kda_commit_mode"):  # the same commit in chunks of 16 rows on the tensor cores
        lib.glm53f_kda_commit_mode.restype, lib.glm53f_kda_commit_mode.argtypes = C.c_int32, [C.c_int32]
        lib.glm53f_kda_commit_mode(1)
        try:
            commit()
            ms_ct = timed(commit)
        finally:
            lib.glm53f_kda_commit_mode(0)
    state_bytes = layers * slots * per * 2
    v_bytes = state_bytes + layers * rows * (TOKEN_IN_BYTES + TOKEN_OUT_BYTES + HEADS * 1284)
    hbm, kind = peaks()
    res = {"workload": f"config 4: {slots} slots x {window} draft rows x {layers} layers, bf16 states, accepted prefixes drawn from 0..{window}",
           "verify": {"ms_per_step": ms_v, "rows_per_s": rows * layers / (ms_v * 1e-3), "state_gbs": state_bytes / (ms_v * 1e-3) / 1e9,
                      "algorithmic_bytes": v_bytes, "gpu_launches": layers,
                      "roofline": {"bound": "hbm", "achieved": v_bytes / (ms_v * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                                   "frac": v_bytes / (ms_v * 1e-3) / 1e9 / hbm, "peak_source": kind,
                                   "counts": "each bf16 state read once, the rows' inputs and outputs, the replay saves written"}},
           "verify_tensor": {"entry": "glm53f_kda_core_verify_batch with GLM53F_KDA_CORE_TENSOR (outputs to bf16-operand rounding, saves and committed states exact)",
                             "ms_per_step": ms_t, "rows_per_s": rows * layers / (ms_t * 1e-3), "state_gbs": state_bytes / (ms_t * 1e-3) / 1e9,
                             "algorithmic_bytes": v_bytes, "gpu_launches": layers,
                             "roofline": {"bound": "hbm", "achieved": v_bytes / (ms_t * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                                          "frac": v_bytes / (ms_t * 1e-3) / 1e9 / hbm, "peak_source": kind}},
           "commit": {"ms_per_step": ms_c, "state_gbs": 2 * state_bytes / (ms_c * 1e-3) / 1e9, "frac_of_hbm": 2 * state_bytes / (ms_c * 1e-3) / 1e9 / hbm,
                      "peak_source": kind, "mean_kept_rows": float(keeps.mean()), "gpu_launches": 1}}
    if ms_ct is not None:
        res["commit_tensor"] = {"entry": "glm53f_kda_core_commit_batch after glm53f_kda_commit_mode(1) (states to the last bits of bf16, not bit for bit)",
                                "ms_per_step": ms_ct, "state_gbs": 2 * state_bytes / (ms_ct * 1e-3) / 1e9,
                                "frac_of_hbm": 2 * state_bytes / (ms_ct * 1e-3) / 1e9 / hbm, "peak_source": kind, "gpu_launches": 1}
    del arena, ks, gs_, vs, bs
    torch.cuda.empty_cache()
    return res


def cpu_marks_gbs(pkg, reps=5):
    """The oracle's copy_mark (numpy row copies through the page list, one host thread) on one whole-model mark."""
    import importlib

    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import rows_oracle as ro

    marks = importlib.import_module(pkg.__name__ + ".marks")
    l = marks.KvLayout.glm53_flash().with_kda_state_bf16(True)
    rng = np.random.default_rng(7)
    parts = [rng.integers(0, 256, r[1], dtype=np.uint8) for r in l.mark_regions()]
    need = l.mark_pages()
    page_list = np.sort(rng.permutation(2 * need)[:need])
    pool = np.zeros(2 * need * l.page_bytes, np.uint8)
    ro.copy_mark(pool, l.page_bytes, page_list, parts, True)
    t0 = time.perf_counter()
    for _ in range(reps):
        ro.copy_mark(pool, l.page_bytes, page_list, parts, True)
        ro.copy_mark(pool, l.page_bytes, page_list, parts, False)
    dt = (time.perf_counter() - t0) / (2 * reps)
    return 2 * l.mark_bytes() / dt / 1e9, 1, f"{2 * reps} copies of one whole-model mark ({l.mark_bytes()} B, {need} pages) by the numpy oracle"


def run_marks(torch, pkg, rank, slots=16, reps=5):
    """The state snapshot of config 1's slots: every slot's positional state of the whole model (34 layers of bf16
    KDA states, the conv windows, the DSA tails: 73.4 MiB) saved into pool pages and restored, one launch per slot
    and direction.  Algorithmic bytes per copy: the mark read once and written once.  `host_api` times GlmKv.mark() +
    rewind() (page allocation and the index upload included); `reference_sequence` the reference's three launches and
    three copies per mark through the same row kernels."""
    import ctypes as C
    import importlib

    import numpy as np

    marks = importlib.import_module(pkg.__name__ + ".marks")
    lib = pkg.ffi.load()
    l = marks.KvLayout.glm53_flash().with_kda_state_bf16(True)
    need = l.mark_pages()
    hbm, kind = peaks()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    res = {"workload": f"{slots} slots x whole-model positional state ({l.mark_bytes()} B = {need} pool pages of {l.page_bytes} B each), "
                       "save into scattered pool pages and restore; 2.3 GiB touched per pass, larger than L2",
           "algorithmic_bytes_per_copy": 2 * l.mark_bytes(), "peak_source": kind}
    for fused in (True, False):
        pool = marks.KvPool(marks.KvConfig(l, slots, slots * need + 64), fused=fused)
        kvs = [pool.slot() for _ in range(slots)]
        pool.state.t.random_(0, 256)
        pool.conv.t.random_(0, 256)
        rng = np.random.default_rng(0x53454544 + rank)
        # scattered pages, as a pool in use hands them out: every mark draws its pages from a shuffle of the pool
        order = rng.permutation(slots * need + 64)
        lists = [torch.tensor(np.sort(order[i * need:(i + 1) * need]).astype(np.int32), device="cuda") for i in range(slots)]
        sizes = (C.c_int64 * 3)(*[n for _, n, _ in l.mark_regions()])

        def device_pass(save):
            for kv, idx in zip(kvs, lists):
                parts = (C.c_void_p * 3)(*[a.as_ptr() + at for a, at in kv._arenas()])
                rc = lib.glm53f_kda_mark_copy(pool.pages.as_ptr(), l.page_bytes, idx.data_ptr(), parts, sizes, save, st)
                if rc != 0:
                    raise RuntimeError(f"mark copy failed: {rc}")

        def api_pass():
            ms = [kv.mark() for kv in kvs]
            for kv, m in zip(kvs, ms):
                kv.rewind(kv.tokens(), m)
            for m in ms:
                m.drop()

        def timed(fn, n):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        if fused:
            for name, save in (("save", 1), ("restore", 0)):
                for _ in range(3):
                    device_pass(save)
                ms = timed(lambda: device_pass(save), reps) / slots
                gbs = 2 * l.mark_bytes() / (ms * 1e-3) / 1e9
                res[name] = {"us_per_mark": ms * 1e3, "gbs": gbs, "frac_of_hbm": gbs / hbm, "gpu_launches_per_mark": 1}
        if fused:
            # all 16 slots' marks by one launch (glm53f_kda_mark_copy_slots)
            all_lists = torch.cat(lists)
            slot_ids = torch.tensor([kv.slot for kv in kvs], dtype=torch.int32, device="cuda")
            arenas = (C.c_void_p * 3)(pool.state.as_ptr(), pool.conv.as_ptr(), pool.tails.as_ptr())
            strides = (C.c_int64 * 3)(l.kda_state_bytes(), l.conv_bytes(), max(l.tails_bytes(), 16))

            def batched(save):
                rc = lib.glm53f_kda_mark_copy_slots(pool.pages.as_ptr(), l.page_bytes, all_lists.data_ptr(), arenas, sizes, strides,
                                                    slot_ids.data_ptr(), slots, save, st)
                if rc != 0:
                    raise RuntimeError(f"mark copy failed: {rc}")

            for name, save in (("save_all_slots_one_launch", 1), ("restore_all_slots_one_launch", 0)):
                for _ in range(3):
                    batched(save)
                ms = timed(lambda: batched(save), reps) / slots
                gbs = 2 * l.mark_bytes() / (ms * 1e-3) / 1e9
                res[name] = {"us_per_mark": ms * 1e3, "gbs": gbs, "frac_of_hbm": gbs / hbm, "gpu_launches": 1}
        for _ in range(2):
            api_pass()
        ms = timed(api_pass, 3) / slots
        res["host_api" if fused else "reference_sequence"] = {"us_per_mark_and_rewind": ms * 1e3, "gbs": 4 * l.mark_bytes() / (ms * 1e-3) / 1e9}
        del pool, kvs, lists
        torch.cuda.empty_cache()
    return res


def run_projections(torch, pkg, rank, layers=6):
    """The GEMMs either side of the KDA core at the model's widths, on the tcgen05 kernel: the fused [q|k|v|b]
    projection 4096 -> 24,640 and o_proj 8192 -> 4096, for a decode step's 16 rows (bound by the weight's bytes: one
    distinct weight per layer, so they stream from HBM) and for a 2,048-row prefill lane (bound by the tensor cores).
    Each shape is a CUDA graph of `layers` launches; the library GEMM (torch.matmul) is timed the same way beside it."""
    import importlib

    proj = importlib.import_module(pkg.__name__ + ".proj")
    g = torch.Generator(device="cuda").manual_seed(0x53454544 + 11 + rank)
    hbm, kind = peaks()
    try:  # a GEMM timed alone: the burst figure of the measured bf16 peak
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf = (float(json.load(f)["bf16_tflops"]), "measured")
    except Exception:
        tf = (1590.0, "fallback")
    res = {"workload": f"x[rows][k] . w[n][k]^T, bf16 in, f32 accumulate, bf16 out; {layers} distinct weights per shape",
           "peak_source": kind, "shapes": []}

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n / layers

    for name, n, k in (("qkvb", proj.KDA_P_COLS, proj.HIDDEN), ("o_proj", proj.HIDDEN, proj.KDA_WIDTH)):
        ws = [(torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(layers)]
        mats = [proj.Bf16Mat.dense(w) for w in ws]
        for rows in (SLOTS, 2048):
            x = torch.randn(rows, k, device="cuda", generator=g).to(torch.bfloat16)
            out = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")

            def ours():
                for m in mats:
                    proj.bf16(x, k, 0, m, rows, out, n, 0)

            def library():
                for w in ws:
                    torch.matmul(x, w.T, out=out)

            ms, ms_lib = timed(ours), timed(library)
            flops, nbytes = 2.0 * rows * n * k, 2.0 * (n * k + rows * (n + k))
            entry = {"gemm": name, "rows": rows, "n": n, "k": k, "us": ms * 1e3, "library_us": ms_lib * 1e3,
                     "tflops": flops / (ms * 1e-3) / 1e12, "gbs": nbytes / (ms * 1e-3) / 1e9, "gpu_launches": 1}
            if rows <= 64:
                entry.update(bound="hbm", frac=entry["gbs"] / hbm, algorithmic_bytes=nbytes)
            else:
                entry.update(bound="tensor", frac=entry["tflops"] / tf[0], peak_tflops=tf[0], tensor_peak_source=tf[1], flops=flops)
            res["shapes"].append(entry)
        del ws, mats
        torch.cuda.empty_cache()
    return res


def run_packed_prefill(torch, pkg, core, rank, passes=10):
    """Config 2: 8,192 rows of packed variable-length sequences (lengths 256..2,048), 64 heads, half of the sequences
    from a carried state: tokens/s per layer through the single-pass kernel (one block per (sequence, head)) and
    through the workspace form."""
    import numpy as np

    lens = pkg.synth.varlen_lengths(2, 8192)
    rows, batch, per = sum(lens), len(lens), STATE_ELEMS
    gen = torch.Generator(device="cuda").manual_seed(0x53454544 + 2 + 97 * rank)
    n = rows * HEADS

    def unit(scale):
        x = torch.randn(n, DK, device="cuda", generator=gen)
        return (x * (scale / torch.sqrt((x * x).sum(1, keepdim=True) + 1e-6))).to(torch.bfloat16).reshape(-1)

    q, k = unit(DK ** -0.5), unit(1.0)
    v = torch.randn(n * DK, device="cuda", generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(n * DK, device="cuda", generator=gen) + 3.0)
    beta = torch.sigmoid(torch.randn(n, device="cuda", generator=gen))
    s0 = torch.zeros(batch * per, device="cuda")
    for i in range(1, batch, 2):
        s0[i * per:(i + 1) * per] = torch.randn(per, device="cuda", generator=gen) * 0.05
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    off = torch.arange(batch, dtype=torch.int64, device="cuda") * per
    out = torch.empty(n * DK, dtype=torch.bfloat16, device="cuda")
    state = s0.clone()
    res = {"workload": f"config 2: {rows} rows in {batch} packed sequences of {min(lens)}..{max(lens)} rows, H=64, d=128, chunk 64, FP32 states"}
    for name, ws in (("single_pass", None), ("workspace", torch.empty(core.prefill_workspace_bytes(HEADS, batch, 32), dtype=torch.uint8, device="cuda"))):
        def once():
            state.copy_(s0)
            core.prefill_varlen(HEADS, rows, cu, max(lens), q, k, v, g, beta, state, off, out=out, workspace=ws)
        for _ in range(3):
            once()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(passes):
            once()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / passes
        res[name] = {"ms_per_layer": ms, "tokens_per_s": rows / (ms * 1e-3), "gbs": rows * PREFILL_BYTES_PER_TOKEN / (ms * 1e-3) / 1e9}
    assert core.device_status() == 0
    return res


PREFILL_T = 1_048_576           # config 3: one sequence, H = 64, d = 128, chunk 64
PREFILL_BYTES_PER_TOKEN = 98_560  # q, k, v, out bf16 + g f32 + beta f32, all 64 heads
PREFILL_FLOP_PER_TOKEN = 8.94e6   # causal-exact count of the chunk-64 form, all 64 heads
BF16_SUSTAINED_TFLOPS_FALLBACK = 1400.0


def tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "measured"
    except Exception:
        return BF16_SUSTAINED_TFLOPS_FALLBACK, "fallback"


def cpu_prefill_toks(seconds: float):
    """The CPU oracle's chunk-64 form on every host core, on a 2,048-token sample of the same distribution."""
    import numpy as np

    o = oracle_module()
    pkg = importlib.import_module("glm53f-afd_b200")
    cores = os.cpu_count() or 1
    t = 2048
    q, k, v, g, b = pkg.synth.tokens(3, 0, t, HEADS)
    s0 = np.zeros(STATE_ELEMS, np.float32)
    n, t0 = 0, time.perf_counter()
    while True:
        o.core_forward(HEADS, q, k, v, g, b, s0, form="chunked", chunk=64, threads=cores, want_y=False)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return n * t / dt, cores, f"{n} x {t} tokens x {HEADS} heads, chunk-64 form, in {dt:.1f} s"


def run_prefill(torch, dist, pkg, core, rank, world, tokens, passes, ws_chunks, check_heads=0):
    """Config 3: chunked prefill of one long sequence, heads sharded over the ranks, outputs all-gathered."""
    import ctypes as C

    par = importlib.import_module("glm53f-afd_b200.parallel")
    lo, hi = par.head_range(HEADS, rank, world)
    hl = hi - lo
    gen = torch.Generator(device="cuda").manual_seed(0x53454544 + 3 + 97 * rank)
    n = tokens * hl
    piece = 1 << 22  # rows of 128 per generation slice: bounds the FP32 temporaries

    def unit(scale):
        out = torch.empty(n * DK, dtype=torch.bfloat16, device="cuda")
        for a in range(0, n, piece):
            m = min(piece, n - a)
            x = torch.randn(m, DK, device="cuda", generator=gen)
            x = x * (scale / torch.sqrt((x * x).sum(1, keepdim=True) + 1e-6))
            out[a * DK:(a + m) * DK] = x.reshape(-1).to(torch.bfloat16)
        return out

    q, k = unit(DK ** -0.5), unit(1.0)
    v = torch.empty(n * DK, dtype=torch.bfloat16, device="cuda")
    g = torch.empty(n * DK, dtype=torch.float32, device="cuda")
    for a in range(0, n, piece):
        m = min(piece, n - a)
        v[a * DK:(a + m) * DK] = torch.randn(m * DK, device="cuda", generator=gen).to(torch.bfloat16)
        g[a * DK:(a + m) * DK] = torch.nn.functional.logsigmoid(torch.randn(m * DK, device="cuda", generator=gen) + 3.0)
    beta = torch.sigmoid(torch.randn(n, device="cuda", generator=gen))
    out = torch.empty(n * DK, dtype=torch.bfloat16, device="cuda")
    state = torch.zeros(hl * DK * DK, device="cuda")
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    off = torch.zeros(1, dtype=torch.int64, device="cuda")
    full = torch.empty((tokens, HEADS, DK), dtype=torch.bfloat16, device="cuda") if world > 1 else None
    # Every rank's full output buffer mapped into every rank: the prefill kernel stores its heads' rows into all of them.
    fused = par.GatheredOutput(tokens, HEADS) if world > 1 else None
    # Few chains (one sequence x this rank's heads): the two-pass form over a workspace keeps every SM busy.  With 32 or
    # fewer chains a workspace that holds every chunk of the sequence lets the kernel cut each chain into segments that
    # are walked at the same time (the scan over segments), which is what shortens the serial walk when heads are sharded.
    if ws_chunks > 0 and world > 1:
        ws_chunks = (tokens + 63) // 64 + 256   # every chunk of the sequence, and the scan's states per super-block
    ws = torch.empty(core.prefill_workspace_bytes(hl, 1, ws_chunks), dtype=torch.uint8, device="cuda") if ws_chunks > 0 else None

    def one_pass(gather):
        """gather: False = this rank's heads only; "nccl" = followed by an all-gather of the outputs; "fused" = the
        kernel stores into every rank's full buffer itself, with a barrier on each side."""
        state.zero_()
        if gather == "fused":
            fused.barrier()
            core.prefill_varlen(hl, tokens, cu, tokens, q, k, v, g, beta, state, off, out=None, workspace=ws,
                                gather=(fused.addresses, HEADS, lo))
            fused.barrier()
            return
        core.prefill_varlen(hl, tokens, cu, tokens, q, k, v, g, beta, state, off, out=out, workspace=ws)
        if gather == "nccl":
            par.gather_heads(out.view(tokens, hl, DK), HEADS, out=full)

    def timed(gather):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(passes):
            one_pass(gather)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / passes
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    one_pass("nccl" if world > 1 else False)
    ms_compute = timed(False)
    ms_nccl = timed("nccl") if world > 1 else ms_compute
    ms_total = ms_compute
    if world > 1:
        if ws is None:
            raise SystemExit("the fused gather needs the workspace form of the prefill (--prefill-ws-chunks > 0)")
        one_pass("fused")
        torch.cuda.synchronize()
        same = torch.equal(fused.tensor.view(torch.int16), full.view(torch.int16))  # both hold the same rows, bit for bit
        ms_total = timed("fused")
    assert core.device_status() == 0
    hbm, hbm_kind = peaks()
    tf, tf_kind = tensor_peak()
    gbs = tokens * PREFILL_BYTES_PER_TOKEN * (hl / HEADS) / (ms_compute * 1e-3) / 1e9      # per GPU
    tflops = tokens * PREFILL_FLOP_PER_TOKEN * (hl / HEADS) / (ms_compute * 1e-3) / 1e12  # per GPU
    chunks = (tokens + 63) // 64
    if world > 1 and ws_chunks > chunks:  # the scan over segments: intra role, two passes of walks, the composition
        kernels_per_pass = 4
    elif ws_chunks >= 2:  # workspace halves: one launch per segment of ws_chunks // 2 chunks, plus the last state role
        kernels_per_pass = (chunks + ws_chunks // 2 - 1) // (ws_chunks // 2) + 1
    else:                 # one chunk per launch pair, or the single-pass kernel
        kernels_per_pass = 2 * chunks if ws_chunks == 1 else 1
    res = {
        "workload": f"config 3: one sequence of {tokens} tokens, H=64 ({hl} heads per GPU), d=128, chunk 64, FP32 state",
        "value": tokens / (ms_total * 1e-3), "unit": "tokens/s per layer", "ms_per_layer": ms_total,
        "heads_per_gpu": hl, "n_gpus": world, "scaling": "strong (the same sequence, heads split over the GPUs)",
        "speedup_hint": HEADS // hl,  # the factor by which this rank's share of the work shrank
        "compute_only": {"value": tokens / (ms_compute * 1e-3), "ms_per_layer": ms_compute},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "peak_source": hbm_kind,
                     "tensor": {"achieved": tflops, "peak": tf, "unit": "TFLOP/s", "frac": tflops / tf, "peak_source": tf_kind,
                                "flop_per_token": PREFILL_FLOP_PER_TOKEN},
                     "algorithmic_bytes_per_token": PREFILL_BYTES_PER_TOKEN,
                     "traffic_bytes_per_token": NCU_PREFILL_DRAM_BYTES_PER_TOKEN if ws_chunks > 0 else None,
                     "kernel": "prefill_sp_kernel (state role + intra role)" if ws_chunks > 0 else "prefill_tc_kernel",
                     "workspace_bytes": 0 if ws is None else ws.numel()},
        "gpu_launches": passes * kernels_per_pass,
        "collective": None if world == 1 else {
            "op": "all-gather of the per-head outputs, fused: the state role stores each output row into every rank's full buffer over NVLink",
            "bytes_sent_per_gpu": tokens * hl * DK * 2 * (world - 1), "ms_exposed": ms_total - ms_compute,
            "equals_nccl_all_gather_bitwise": bool(same),
            "nccl_all_gather_after_the_kernel": {"ms_per_layer": ms_nccl, "ms_exposed": ms_nccl - ms_compute}},
    }
    if check_heads > 0 and rank == 0:
        res["check"] = check_prefill(torch, tokens, hl, min(check_heads, hl), q, k, v, g, beta, out, state)
    del q, k, v, g, out, full, fused
    torch.cuda.empty_cache()
    return res


def check_prefill(torch, tokens, hl, n_heads, q, k, v, g, beta, out, state):
    """Full-length parity of the prefill leg: the FP32 row-by-row recurrence of the oracle on the host, from the exact
    bytes the GPU consumed, for `n_heads` heads spread over this rank's heads: final-state rel-L2 and the outputs of
    the last 4,096 tokens (max-abs and rel-L2 against the FP32 read-out)."""
    import numpy as np

    o = oracle_module()
    sel = sorted({(i * hl) // n_heads for i in range(n_heads)})
    idx = torch.tensor(sel, device="cuda")
    pick = lambda t, w: t.view(tokens, hl, w).index_select(1, idx).contiguous().cpu()
    qh, kh, vh = (pick(t.view(torch.int16), DK).numpy().view(np.uint16).reshape(-1) for t in (q, k, v))
    gh = pick(g, DK).numpy().reshape(-1)
    bh = beta.view(tokens, hl).index_select(1, idx).contiguous().cpu().numpy().reshape(-1)
    t0 = time.perf_counter()
    y, s_ref = o.core_forward(len(sel), qh, kh, vh, gh, bh, np.zeros(len(sel) * DK * DK, np.float32), form="recurrent",
                              threads=min(len(sel), os.cpu_count() or 1))
    cpu_s = time.perf_counter() - t0
    s_gpu = state.view(hl, DK * DK).index_select(0, idx).cpu().numpy().reshape(-1)
    tail = min(tokens, 4096)
    y_gpu = out.view(tokens, hl, DK)[tokens - tail:].index_select(1, idx).float().cpu().numpy().reshape(-1)
    y_ref = y.reshape(tokens, len(sel), DK)[tokens - tail:].reshape(-1)
    return {"heads": sel, "tokens": tokens, "state_rel_l2": float(np.linalg.norm(s_gpu - s_ref) / np.linalg.norm(s_ref)),
            "out_tail_tokens": tail, "out_max_abs": float(np.max(np.abs(y_gpu - y_ref))),
            "out_rel_l2": float(np.linalg.norm(y_gpu - y_ref) / np.linalg.norm(y_ref)),
            "limits": {"state_rel_l2": 1e-3, "out_max_abs": 2e-2, "out_rel_l2": 5e-3}, "cpu_seconds": cpu_s}


def run_decode_strong(torch, dist, lib, rank, world, layers, steps):
    """The benchmark's own sharding of configurations 1 and 4: a fixed number of slots (16, 48) split by slot over the
    ranks (no collective), every rank's 34 layer launches replayed from one CUDA graph; whole-job state GB/s from the
    slowest rank.  With 8 GPUs a rank holds 2 (6) slots: the launches are short and the figure shows what that costs."""
    par = importlib.import_module("glm53f-afd_b200.parallel")
    res = []
    for total in (SLOTS, VERIFY_SLOTS):
        lo, hi = par.slot_range(total, rank, world)
        n = hi - lo
        gen = torch.Generator(device="cuda").manual_seed(0x53454544 + 41 + rank)
        rows = n * HEADS

        def unit(scale):
            x = torch.randn(rows, DK, device="cuda", generator=gen)
            return (x * (scale / torch.sqrt((x * x).sum(1, keepdim=True) + 1e-6))).to(torch.bfloat16).reshape(-1)

        q, k = unit(DK ** -0.5), unit(1.0)
        v = torch.randn(rows * DK, device="cuda", generator=gen).to(torch.bfloat16)
        g = torch.nn.functional.logsigmoid(torch.randn(rows * DK, device="cuda", generator=gen) + 3.0)
        beta = torch.sigmoid(torch.randn(rows, device="cuda", generator=gen))
        arena = (torch.randn(layers * n * STATE_ELEMS, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
        out = torch.empty(rows * DK, dtype=torch.bfloat16, device="cuda")
        cu = torch.arange(n + 1, dtype=torch.int32, device="cuda")
        offs = torch.arange(n, dtype=torch.int64, device="cuda") * STATE_ELEMS
        P = lambda t: C.c_void_p(t.data_ptr())

        def step(stream):
            for l in range(layers):
                st = C.c_void_p(arena.data_ptr() + 2 * l * n * STATE_ELEMS)
                rc = lib.glm53f_kda_core_decode_batch(HEADS, n, P(cu), P(q), P(k), P(v), P(g), P(beta), st, st, P(offs), 1, 0, None, None, 1e-5, P(out), stream)
                if rc != 0:
                    raise RuntimeError(f"decode launch failed: {rc}")

        _ms, graph = graph_ms(torch, step, 3)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        gbs = layers * total * STATE_ELEMS * 4 / (ms * 1e-3) / 1e9
        res.append({"slots_total": total, "slots_per_gpu": n, "ms_per_step": ms, "state_gbs": gbs, "us_per_launch": ms * 1e3 / layers,
                    "gpu_launches": steps * layers})
        del arena, graph, q, k, v, g, beta, out
        torch.cuda.empty_cache()
    return res


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def headline_config(layers):
    return {"workload": "config 1: batched single-token decode, 16 slots per GPU, H=64, d=128, 34 layers, bf16-stored states",
            "layers": layers, "l2": "inputs larger than L2: 1.06 GiB of states stream per step", "sharding": "by slot, no collective",
            "launch": "one CUDA graph of the step's 34 launches, replayed"}


METRIC = "KDA decode state GB/s (16 slots x 34 layers, bf16 states)"


def bind_to_gpu_numa(torch, index):
    """Best effort: run this process on the CPUs of the GPU's NUMA node, so that pinned staging buffers are local to the
    GPU's PCIe root (first touch).  Returns the node, or None when the topology files say nothing."""
    try:
        bus = torch.cuda.get_device_properties(index).pci_bus_id
        dom = torch.cuda.get_device_properties(index).pci_domain_id
        dev = torch.cuda.get_device_properties(index).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def e2e_stepper(torch, layers, layer_in, out_bytes, host_in, dev_in, dev_out, host_out, launch_layer, group=9):
    """One end-to-end step: the step's inputs go from one pinned host block to the device in a few large copies, one
    per group of layers on a copy stream, so that the transfer of the next group runs beside the launches of the
    current one; the outputs come back the same way; the step ends when its outputs are on the host.  (34 layers with
    group = 9: groups of 9, 9, 8, 4, 2, 1, 1 layers.)"""
    # Groups of `group` layers while many layers remain, then halving down to one: the host-to-device pipe is the
    # bottleneck, so what a step adds to the transfer time is the work left once the LAST group's inputs have arrived,
    # and a last group of one layer makes that one launch and one small copy back.
    groups, a = [], 0
    while a < layers:
        left = layers - a
        n = 1 if left == 1 else min(group, max(1, left // 2))
        groups.append((a, a + n))
        a += n
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step():
        main = torch.cuda.current_stream()
        copy_in.wait_stream(main)   # the previous step's launches have read the staging block
        copy_out.wait_stream(main)
        for a, b in groups:
            with torch.cuda.stream(copy_in):
                dev_in[a * layer_in:b * layer_in].copy_(host_in[a * layer_in:b * layer_in], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record()
            main.wait_event(arrived)
            for l in range(a, b):
                launch_layer(l)
            done = torch.cuda.Event()
            done.record()
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                host_out[a * out_bytes:b * out_bytes].copy_(dev_out[a * out_bytes:b * out_bytes], non_blocking=True)
        main.wait_stream(copy_out)

    return step


def run_reference_cpu(args):
    """No reference kernels and no GPU needed: the reference's CPU formulation (the oracle port) on the host cores."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    per_step = max(1.0, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_decode_gbs(min(per_step, 1.0))
    vals = []
    for _ in range(args.steps):
        v, cores, sample = cpu_decode_gbs(per_step)
        vals.append(v)
    value = sum(vals) / len(vals)
    ms = STATE_BYTES_PER_LAUNCH * LAYERS / (value * 1e9) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(LAYERS),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "oracle/_ref (the reference's own kernels) is absent: this is the reference's CPU formulation, the C++ port in oracle/ "
                "(its own CPU code is Rust, no toolchain here), all host threads, a bounded number of repetitions of 2 of the 34 layers",
    }
    print(json.dumps(line), flush=True)


def run_reference(args):
    """The reference arm: the reference's own CUDA kernels (oracle/_ref, compiled unmodified from the reference tree) on
    this GPU, entered through the symbol its forward calls for a decode step (glm53f_kda_chain_batch_bf16state,
    crates/glm53f-forward/src/forward.rs:3672-3735) with the forward's argument values; same slots, heads, layers,
    distinct states per layer, CUDA graph of the step's launches, event timing, and the same end-to-end loop (the
    step's projection rows and gate rows from pinned host memory, the outputs back).  Every rank runs its own 16
    slots, as in the product arm."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    pkg = importlib.import_module("glm53f-afd_b200")
    ref = reference_library(pkg) if has_gpu else None
    if ref is None:
        return run_reference_cpu(args)
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    numa = bind_to_gpu_numa(torch, local_rank)
    layers = args.layers
    d = LayerAbi(torch, rank, SLOTS, 1, layers)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _ms, graph = graph_ms(torch, lambda st: [d.chain(ref, l, st) for l in range(layers)], max(3, args.warmup))
    t_c0 = time.time()
    ms = timed(graph.replay, args.steps)
    t_c1 = time.time()
    while time.time() < t_c1 + 0.4:   # untimed: the same graph under the clock sampler
        graph.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop(t_c0, time.time(), t_c1) if rank == 0 else None
    ms_per_step = ms / args.steps
    per_rank_bytes = layers * STATE_BYTES_PER_LAUNCH
    value = world * per_rank_bytes / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = peaks()
    achieved = STATE_BYTES_PER_LAUNCH / (ms * 1e-3 / (args.steps * layers)) / 1e9
    # end to end
    layer_in, out_bytes = SLOTS * LAYER_IN_BYTES, SLOTS * OUT_STRIDE * 2
    host_in = torch.empty(layers * layer_in, dtype=torch.uint8).pin_memory()
    host_in.random_(0, 64)
    dev_in = torch.empty(layers * layer_in, dtype=torch.uint8, device="cuda")
    dev_in.copy_(host_in)
    dev_out = torch.empty(layers * out_bytes, dtype=torch.uint8, device="cuda")
    host_out = torch.empty(layers * out_bytes, dtype=torch.uint8).pin_memory()
    in16, out16 = dev_in.view(torch.bfloat16), dev_out.view(torch.bfloat16)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    le = layer_in // 2

    def launch_layer(l):
        d.chain(ref, l, stream, p=d.at(in16, l * le), ag=(in16, l * le + SLOTS * P_STRIDE), out=d.at(out16, l * out_bytes // 2))

    e2e_step = e2e_stepper(torch, layers, layer_in, out_bytes, host_in, dev_in, dev_out, host_out, launch_layer)
    for _ in range(3):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps) / args.steps
    e2e_value = world * per_rank_bytes / (e2e_ms * 1e-3) / 1e9
    del d, graph, dev_in, dev_out
    torch.cuda.empty_cache()
    shapes = run_layer_abi(torch, ref, rank, layers, args.steps) if (rank == 0 and not args.no_verify) else None
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": headline_config(layers),
        "reference_kind": "the reference's own CUDA kernels (crates/glm53f-kda/kernels/kda.cu, kda_prefill.cu) compiled unmodified for sm_100a, on this GPU",
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": peak_kind, "kernel": "the reference's chain_kernel<bf16>"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": layers * SLOTS * LAYER_IN_BYTES,
                "d2h_bytes_per_step": layers * SLOTS * TOKEN_OUT_BYTES, "numa_node": numa},
        "gpu_launches": args.steps * layers, "clocks": clocks, "layer_abi": shapes,
    }
    if not args.no_cpu:
        v, cores, sample = cpu_decode_gbs(args.cpu_seconds)
        line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=8.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers per step (profiling runs use fewer)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_T, help="sequence length of the prefill leg (0 skips it)")
    ap.add_argument("--prefill-passes", type=int, default=3)
    ap.add_argument("--no-proj", action="store_true", help="skip the projection GEMM leg")
    ap.add_argument("--no-marks", action="store_true", help="skip the state snapshot / restore leg")
    ap.add_argument("--no-verify", action="store_true", help="skip the draft-verification leg (config 4) and the packed-prefill leg (config 2)")
    ap.add_argument("--prefill-check-heads", type=int, default=-1, help="check this many heads of the prefill leg at full length against the CPU recurrence (about half a minute per head and core at 1M tokens); default: 4 on one GPU, 0 under torchrun")
    ap.add_argument("--e2e-group", type=int, default=9, help="layers per host-to-device copy of the end-to-end step")
    ap.add_argument("--prefill-ws-chunks", type=int, default=256, help="chunks of 64 rows per pass of the two-pass prefill (0: single-pass kernel)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch

    dist = None
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    numa = bind_to_gpu_numa(torch, local_rank)  # before any pinned allocation: staging is first touched on the GPU's node
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # early: it is running long before the timed region
    pkg = importlib.import_module("glm53f-afd_b200")
    core = importlib.import_module("glm53f-afd_b200.core")
    ffi = pkg.ffi
    lib = ffi.load()  # raises when the CUDA library is missing: there is no fallback
    layers = args.layers
    if args.prefill_check_heads < 0:
        args.prefill_check_heads = 4 if world == 1 else 0

    # ---- inputs: host-generated tokens (seeded, exact distributions), device-generated carried states N(0, 0.05)
    gen = torch.Generator(device="cuda").manual_seed(0x53454544 + 1 + rank)
    arena = (torch.randn(layers * SLOTS * STATE_ELEMS, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    host = []
    for l in range(layers):
        q, k, v, g, b = pkg.synth.tokens(1, l + 1000 * rank, SLOTS, HEADS)
        host.append([torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).pin_memory() for x in (q, k, v, g, b)])
    dev = [[t.cuda() for t in ts] for ts in host]
    outs = [torch.zeros(SLOTS * HEADS * DK, dtype=torch.int16, device="cuda") for _ in range(layers)]
    cu = torch.arange(SLOTS + 1, dtype=torch.int32, device="cuda")
    offs = torch.arange(SLOTS, dtype=torch.int64, device="cuda") * STATE_ELEMS
    # one checked launch, then raw calls in the timed loops (as the reference's own bench does)
    core.decode_batch(HEADS, SLOTS, cu, *dev[0], arena[:SLOTS * STATE_ELEMS], offs, out=outs[0])
    torch.cuda.synchronize()
    assert core.device_status() == 0
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: C.c_void_p(t.data_ptr())

    def step(inputs):
        for l in range(layers):
            q, k, v, g, b = inputs[l]
            st = C.c_void_p(arena.data_ptr() + 2 * l * SLOTS * STATE_ELEMS)
            rc = lib.glm53f_kda_core_decode_batch(HEADS, SLOTS, P(cu), P(q), P(k), P(v), P(g), P(b), st, st, P(offs), 1, 0, None,
                                                  None, 1e-5, P(outs[l]), stream)
            if rc != 0:
                raise RuntimeError(f"decode launch failed: {rc}")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    # ---- device-resident timing: the step's 34 launches are captured once in a CUDA graph and replayed, as a serving
    # loop would (the entry points read their batch metadata on the device, so a captured step can be replayed).
    for _ in range(max(3, args.warmup)):
        step(dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    stream = C.c_void_p(side.cuda_stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step(dev)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step(dev)
    torch.cuda.synchronize()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        graph.replay()
    t_c0 = time.time()
    ms = timed(graph.replay, args.steps)
    timed_launches = args.steps * layers
    t_c1 = time.time()
    while time.time() < t_c1 + 0.4:   # untimed: the same graph under the clock sampler
        graph.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop(t_c0, time.time(), t_c1) if rank == 0 else None
    ms_per_step = ms / args.steps
    per_rank_bytes = layers * STATE_BYTES_PER_LAUNCH
    value = world * per_rank_bytes / (ms_per_step * 1e-3) / 1e9
    launch_s = ms * 1e-3 / (args.steps * layers)
    achieved = STATE_BYTES_PER_LAUNCH / launch_s / 1e9
    peak, peak_kind = peaks()

    # ---- end to end: pinned host inputs in, outputs back, every step.  The step's inputs live in one pinned host
    # block (as an engine would stage a step's activations) and go over in a few large copies, one per group of
    # layers on a copy stream, so that the transfer of the next group runs beside the launches of the current one;
    # the outputs come back the same way.
    in_elems = [t.numel() * t.element_size() for t in host[0]]
    layer_in = sum(in_elems)
    out_bytes = SLOTS * HEADS * DK * 2
    host_in = torch.empty(layers * layer_in, dtype=torch.uint8).pin_memory()
    dev_in = torch.empty(layers * layer_in, dtype=torch.uint8, device="cuda")
    dev_out = torch.empty(layers * out_bytes, dtype=torch.uint8, device="cuda")
    host_out = torch.empty(layers * out_bytes, dtype=torch.uint8).pin_memory()
    staged = []
    for l in range(layers):
        at, views = l * layer_in, []
        for t, nb in zip(host[l], in_elems):
            host_in[at:at + nb].copy_(t.view(torch.uint8).reshape(-1))
            views.append(dev_in[at:at + nb].view(t.dtype))
            at += nb
        staged.append(views)
    e2e_outs = [dev_out[l * out_bytes:(l + 1) * out_bytes].view(torch.int16) for l in range(layers)]
    def launch_layer(l):
        q, k, v, g, bb = staged[l]
        st = C.c_void_p(arena.data_ptr() + 2 * l * SLOTS * STATE_ELEMS)
        rc = lib.glm53f_kda_core_decode_batch(HEADS, SLOTS, P(cu), P(q), P(k), P(v), P(g), P(bb), st, st, P(offs), 1, 0, None,
                                              None, 1e-5, P(e2e_outs[l]), stream)
        if rc != 0:
            raise RuntimeError(f"decode launch failed: {rc}")

    e2e_step = e2e_stepper(torch, layers, layer_in, out_bytes, host_in, dev_in, dev_out, host_out, launch_layer, group=args.e2e_group)
    for _ in range(3):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps) / args.steps
    e2e_value = world * per_rank_bytes / (e2e_ms * 1e-3) / 1e9
    assert core.device_status() == 0

    del arena, dev, outs, dev_in, dev_out, staged, e2e_outs
    torch.cuda.empty_cache()
    verify = run_verify(torch, lib, rank, layers, max(3, args.steps // 4)) if not args.no_verify else None
    assert core.device_status() == 0
    packed = run_packed_prefill(torch, pkg, core, rank) if not args.no_verify else None
    marks = run_marks(torch, pkg, rank) if not args.no_marks else None
    projections = run_projections(torch, pkg, rank) if not args.no_proj else None
    strong = run_decode_strong(torch, dist if world > 1 else None, lib, rank, world, layers, args.steps) if not args.no_verify else None
    layer_abi = run_layer_abi(torch, lib, rank, layers, args.steps) if (rank == 0 and not args.no_verify) else None
    assert core.device_status() == 0
    prefill = None
    if args.prefill_tokens > 0:
        prefill = run_prefill(torch, dist if world > 1 else None, pkg, core, rank, world, args.prefill_tokens, args.prefill_passes, args.prefill_ws_chunks, args.prefill_check_heads)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    line = {
        "metric": METRIC,
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": headline_config(layers),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "peak_source": peak_kind, "frac_of_nominal_8tbs": achieved / 8000.0,
                     "algorithmic_bytes_per_launch": STATE_BYTES_PER_LAUNCH, "kernel": "recurrent_kernel<bf16, core>"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": layers * SLOTS * TOKEN_IN_BYTES,
                "d2h_bytes_per_step": layers * SLOTS * TOKEN_OUT_BYTES, "numa_node": numa,
                "h2d_plus_d2h_gbs_per_rank": layers * SLOTS * (TOKEN_IN_BYTES + TOKEN_OUT_BYTES) / (e2e_ms * 1e-3) / 1e9},
        "gpu_launches": timed_launches,
        "clocks": clocks,
        "verify": verify,
        "decode_strong": strong,
        "layer_abi": layer_abi,
        "prefill_packed": packed,
        "marks": marks,
        "projections": projections,
        "prefill": prefill,
    }
    if not args.no_cpu:
        v, cores, sample = cpu_decode_gbs(args.cpu_seconds)
        line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
        if marks is not None:
            v, cores, sample = cpu_marks_gbs(pkg)
            marks["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
        if prefill is not None:
            v, cores, sample = cpu_prefill_toks(args.cpu_seconds)
            prefill["cpu_baseline"] = {"value": v, "unit": "tokens/s per layer", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
