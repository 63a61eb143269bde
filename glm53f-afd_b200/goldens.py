"""Golden-fixture sets of the reference model (the transformers reference run on the checkpoint) and the checks of the
KDA core against them.

Mirror of crates/glm53f-kda/src/goldens.rs: the set format (`manifest.json` with one member per tensor -- file, dtype,
shape, sha256 -- beside raw little-endian `.bin` payloads; goldens.rs:182-240), digest and size verification on every
read (277-301), the mapping from the oracle's tensor names to roles (413-543), the per-layer grouping (545-597), the
comparison and its tolerance tiers relative to max |ref| (642-761: f32 1e-4, bf16 recurrent 1e-2, bf16 chunked 5e-2) and
`check_core` (885-955), which here runs the B200 kernels instead of the CPU recurrence.  The payloads themselves are
not in the reference repository (they need the checkpoint); `write_set` (1276-1310) makes sets for tests.
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

DK = DV = 128
DECODER_LAYERS = 45  # lib.rs:58

TOL_F32 = 1e-4        # goldens.rs:756
TOL_RECURRENT = 1e-2  # goldens.rs:758
TOL_CHUNKED = 5e-2    # goldens.rs:761


def is_kda_layer(i: int) -> bool:
    """Every fourth layer is full attention; the others run KDA (lib.rs:68-70)."""
    return i < DECODER_LAYERS and i % 4 != 3


class GoldenError(Exception):
    """kind: "io", "json", "manifest", "digest", "size", "missing" or "shape" (goldens.rs:47-68)."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


class DType(enum.Enum):
    F64 = ("f64", 8, "<f8")
    F32 = ("f32", 4, "<f4")
    F16 = ("f16", 2, "<f2")
    BF16 = ("bf16", 2, "<u2")
    I64 = ("i64", 8, "<i8")
    I32 = ("i32", 4, "<i4")
    U8 = ("u8", 1, "u1")

    @staticmethod
    def parse(s: str) -> Optional["DType"]:
        key = s.lower()
        if key.startswith("torch."):
            key = key[6:]
        table = {"f64": DType.F64, "float64": DType.F64, "double": DType.F64, "f32": DType.F32, "float32": DType.F32, "float": DType.F32,
                 "f16": DType.F16, "float16": DType.F16, "half": DType.F16, "bf16": DType.BF16, "bfloat16": DType.BF16,
                 "i64": DType.I64, "int64": DType.I64, "long": DType.I64, "i32": DType.I32, "int32": DType.I32, "int": DType.I32,
                 "u8": DType.U8, "uint8": DType.U8, "bool": DType.U8}
        return table.get(key)

    def size(self) -> int:
        return self.value[1]

    def manifest_name(self) -> str:
        return self.value[0]


@dataclass
class Entry:
    name: str
    file: str
    dtype: DType
    shape: list
    sha256: str

    def elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass
class Tensor:
    """A fixture widened to f32 (as the reference reads them), with its stored dtype and shape."""

    name: str
    dtype: DType
    shape: list
    data: np.ndarray


class Phase(enum.Enum):
    Prefill = "prefill"
    Decode = "decode"


def _bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


class Set:
    """One fixture set: a directory with manifest.json and the payloads it names (goldens.rs:182-387)."""

    def __init__(self, directory: str, entries: list, notes):
        self.dir, self.entries, self.notes = directory, entries, notes

    @classmethod
    def load(cls, directory: str) -> "Set":
        path = os.path.join(directory, "manifest.json")
        try:
            with open(path) as f:
                text = f.read()
        except OSError as e:
            raise GoldenError("io", f"{path}: {e}")
        try:
            doc = json.loads(text)
        except ValueError as e:
            raise GoldenError("json", f"{path}: {e}")
        members = doc.get("tensors", doc) if isinstance(doc, dict) else None
        if not isinstance(members, dict):
            raise GoldenError("manifest", "not a JSON object")
        entries = []
        for name, v in members.items():
            if not isinstance(v, dict) or not isinstance(v.get("file"), str):
                continue  # other members are metadata; tensor entries have a "file"
            bad = lambda what: GoldenError("manifest", f"{name}: {what}")
            if not isinstance(v.get("dtype"), str):
                raise bad("no dtype")
            dtype = DType.parse(v["dtype"])
            if dtype is None:
                raise bad("unknown dtype")
            shape = v.get("shape")
            if not isinstance(shape, list):
                raise bad("no shape")
            if not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape):
                raise bad("bad shape")
            if not isinstance(v.get("sha256"), str):
                raise bad("no sha256")
            file = v["file"]
            if ".." in file or file.startswith("/"):
                raise bad("file must stay inside the set")
            entries.append(Entry(name, file, dtype, list(shape), v["sha256"].lower()))
        return cls(directory, entries, doc.get("notes") if isinstance(doc, dict) else None)

    def name(self) -> str:
        return os.path.basename(os.path.normpath(self.dir))

    def layer_phase(self):
        """("layerNN-prefill" | "layerNN-decode") -> (NN, Phase), else None."""
        n = self.name()
        if not n.startswith("layer") or "-" not in n:
            return None
        layer, phase = n[5:].split("-", 1)
        if not layer.isdigit() or phase not in ("prefill", "decode"):
            return None
        return int(layer), Phase(phase)

    def state_heads(self):
        if isinstance(self.notes, dict) and isinstance(self.notes.get("state_heads"), list):
            hs = self.notes["state_heads"]
            if all(isinstance(h, int) and h >= 0 for h in hs):
                return list(hs)
        return None

    def entry(self, name: str) -> Optional[Entry]:
        return next((e for e in self.entries if e.name == name), None)

    def bytes(self, name: str) -> bytes:
        """The payload, after its size and SHA-256 matched the manifest."""
        e = self.entry(name)
        if e is None:
            raise GoldenError("missing", name)
        path = os.path.join(self.dir, e.file)
        try:
            with open(path, "rb") as f:
                data = f.read()
        except OSError as err:
            raise GoldenError("io", f"{path}: {err}")
        expected = e.elements() * e.dtype.size()
        if len(data) != expected:
            raise GoldenError("size", f"{name}: {len(data)} bytes, expected {expected}")
        actual = hashlib.sha256(data).hexdigest()
        if actual != e.sha256:
            raise GoldenError("digest", f"{name}: sha256 {actual}, manifest says {e.sha256}")
        return data

    def read(self, name: str) -> Tensor:
        e = self.entry(name)
        if e is None:
            raise GoldenError("missing", name)
        raw = np.frombuffer(self.bytes(name), dtype=np.dtype(e.dtype.value[2]))
        data = _bf16_to_f32(raw) if e.dtype is DType.BF16 else raw.astype(np.float32)
        return Tensor(e.name, e.dtype, list(e.shape), np.ascontiguousarray(data))

    def verify_all(self) -> None:
        for e in self.entries:
            self.bytes(e.name)


def default_root() -> str:
    """$GLM53F_GOLDENS, else oracle/goldens of a reference checkout given by $GLM53F_REFERENCE (goldens.rs:389-395)."""
    if os.environ.get("GLM53F_GOLDENS"):
        return os.environ["GLM53F_GOLDENS"]
    return os.path.join(os.environ.get("GLM53F_REFERENCE", "."), "oracle", "goldens")


def discover(root: str) -> list:
    """The sets under root (subdirectories with a manifest.json), sorted; empty when root does not exist."""
    try:
        names = sorted(os.listdir(root))
    except OSError:
        return []
    return [os.path.join(root, n) for n in names if os.path.isfile(os.path.join(root, n, "manifest.json"))]


class Role(enum.Enum):
    Q = "q"
    K = "k"
    V = "v"
    LogDecay = "log_decay"
    Beta = "beta"
    StateIn = "state_in"
    StateOut = "state_out"
    StateSteps = "state_steps"
    CoreOut = "core_out"
    Path = "path"
    MixedQkv = "mixed_qkv"
    ConvStateIn = "conv_state_in"
    ConvStateOut = "conv_state_out"
    ForgetProj = "forget_proj"
    BetaLogits = "beta_logits"
    GateProj = "gate_proj"
    NormOut = "norm_out"
    ConvW = "conv_w"
    ConvWQ = "conv_w_q"
    ConvWK = "conv_w_k"
    ConvWV = "conv_w_v"
    ALog = "a_log"
    DtBias = "dt_bias"
    NormW = "norm_w"


# goldens.rs:460-499
ROLES = [
    (Role.Q, ("q", "query")), (Role.K, ("k", "key")), (Role.V, ("v", "value")), (Role.LogDecay, ("g", "log_decay")), (Role.Beta, ("beta",)),
    (Role.StateIn, ("initial_state", "state_in")),
    (Role.StateOut, ("state", "state_final", "final_state", "state_out", "last_recurrent_state")),
    (Role.StateSteps, ("state_heads",)), (Role.CoreOut, ("core_out", "core_attn_out")), (Role.Path, ("path",)),
    (Role.MixedQkv, ("qkv_preconv", "mixed_qkv")), (Role.ConvStateIn, ("conv_state_in",)),
    (Role.ConvStateOut, ("conv_state", "conv_state_final", "conv_state_out")),
    (Role.ForgetProj, ("f_proj", "forget_proj", "f_b_proj")), (Role.BetaLogits, ("b_logits", "b_proj", "beta_logits")),
    (Role.GateProj, ("gate", "g_proj", "g_b_proj")), (Role.NormOut, ("norm_out", "o_norm_out")),
    (Role.ConvW, ("conv1d.weight", "conv_w")), (Role.ConvWQ, ("q_conv1d.weight",)), (Role.ConvWK, ("k_conv1d.weight",)),
    (Role.ConvWV, ("v_conv1d.weight",)), (Role.ALog, ("a_log",)), (Role.DtBias, ("dt_bias",)), (Role.NormW, ("o_norm.weight", "norm_w")),
]
MODULES = ("weights", "kda", "self_attn", "linear_attn", "forget_gate")


def classify(name: str, set_layer: Optional[int]):
    """(layer, role) of a tensor name, or None (goldens.rs:503-543).  The layer is a `layers.N` / `layerN` / `LNN`
    component of the name, else the set's own layer; per-step tensors (`decode.sN.*`) and non-KDA layers are skipped."""
    parts = name.lower().replace("/", ".").split(".")
    if parts and parts[0] in ("prefill", "decode"):
        parts = parts[1:]
        if parts and len(parts[0]) > 1 and parts[0][0] == "s" and parts[0][1:].isdigit():
            return None
    found = None
    for i, p in enumerate(parts):
        digits = p[5:] if p.startswith("layer") else (p[1:] if p.startswith("l") else p)
        if digits and digits.isdigit() and digits.isascii():
            found = (i, int(digits))
            break
    if found is not None:
        rest, layer = parts[found[0] + 1:], found[1]
    elif set_layer is not None:
        rest, layer = parts, set_layer
    else:
        return None
    if not is_kda_layer(layer):
        return None
    key = ".".join(p for p in rest if p not in MODULES)
    for role, names in ROLES:
        if key in names:
            return layer, role
    return None


@dataclass
class LayerFixtures:
    layer: int
    phase: Optional[Phase]
    tensors: list = field(default_factory=list)  # (role, tensor name), the first name seen per role

    def name(self, role: Role) -> Optional[str]:
        return next((n for r, n in self.tensors if r is role), None)

    def has(self, roles) -> bool:
        return all(self.name(r) is not None for r in roles)


def kda_layers(s: Set) -> list:
    lp = s.layer_phase()
    set_layer, phase = (lp[0], lp[1]) if lp else (None, None)
    layers: list = []
    for e in s.entries:
        c = classify(e.name, set_layer)
        if c is None:
            continue
        layer, role = c
        lf = next((l for l in layers if l.layer == layer), None)
        if lf is None:
            layers.append(LayerFixtures(layer, phase if layer == set_layer else None, [(role, e.name)]))
        elif lf.name(role) is None:
            lf.tensors.append((role, e.name))
    layers.sort(key=lambda l: l.layer)
    return layers


@dataclass
class Init:
    """What a decode set starts from: the state and conv window its layer's prefill set ended with (goldens.rs:599-640)."""

    state: Optional[np.ndarray] = None
    conv: Optional[np.ndarray] = None

    @classmethod
    def from_prefill(cls, s: Set, layer: int) -> "Init":
        if s.layer_phase() != (layer, Phase.Decode):
            return cls()
        directory = os.path.join(os.path.dirname(os.path.normpath(s.dir)), f"layer{layer:02d}-prefill")
        if not os.path.isfile(os.path.join(directory, "manifest.json")):
            return cls()
        prefill = Set.load(directory)
        lf = next((l for l in kda_layers(prefill) if l.layer == layer), None)
        if lf is None:
            return cls()
        read = lambda role: prefill.read(lf.name(role)).data if lf.name(role) else None
        return cls(read(Role.StateOut), read(Role.ConvStateOut))


class Weight(enum.Enum):
    Required = "required"
    Informational = "informational"


@dataclass
class Comparison:
    """goldens.rs:642-754: max |diff| against tol * max(max |ref|, 1e-3)."""

    what: str
    elements: int
    max_abs: float
    max_ref: float
    max_ulp: int
    differing: int
    tol: float
    weight: Weight = Weight.Required

    @classmethod
    def compare(cls, what: str, got, want, tol: float) -> "Comparison":
        got = np.ascontiguousarray(got, dtype=np.float32).reshape(-1)
        want = np.ascontiguousarray(want, dtype=np.float32).reshape(-1)
        if got.size != want.size:
            raise GoldenError("shape", f"{what}: {got.size} elements against {want.size}")
        d = np.abs(got - want)
        max_abs = float("inf") if np.isnan(d).any() else float(d.max(initial=0.0))
        a, b = _f32_to_bf16(got).astype(np.int64), _f32_to_bf16(want).astype(np.int64)
        key = lambda u: np.where(u & 0x8000, 0x8000 - (u & 0x7FFF), 0x8000 + u)  # sign-magnitude to a monotone scale
        max_ulp = int(np.abs(key(a) - key(b)).max(initial=0))
        return cls(what, int(got.size), max_abs, float(np.abs(want).max(initial=0.0)), max_ulp,
                   int((got.view(np.uint32) != want.view(np.uint32)).sum()), tol)

    def passes(self) -> bool:
        return self.max_abs <= self.tol * max(self.max_ref, 1e-3)

    def __str__(self) -> str:
        tail = "" if self.weight is Weight.Required else " [reported only]"
        return (f"{self.what}: {self.elements} elements, max |diff| {self.max_abs:.3e} (max |ref| {self.max_ref:.3e}, tolerance "
                f"{self.tol:.1e} relative), max {self.max_ulp} bf16 ulp, {self.differing} differ{tail}")


def verdict(results) -> bool:
    return all(c.passes() for c in results if c.weight is Weight.Required)


def tolerance(dtype: DType, recurrent: bool) -> float:
    if dtype in (DType.F32, DType.F64):
        return TOL_F32
    return TOL_RECURRENT if recurrent else TOL_CHUNKED


def _tensor(s: Set, lf: LayerFixtures, role: Role) -> Tensor:
    name = lf.name(role)
    if name is None:
        raise GoldenError("missing", f"layer {lf.layer} {role.name}")
    return s.read(name)


def _optional(s: Set, lf: LayerFixtures, role: Role) -> Optional[Tensor]:
    return _tensor(s, lf, role) if lf.name(role) else None


def _expect_len(t: Tensor, n: int) -> None:
    if t.data.size != n:
        raise GoldenError("shape", f"{t.name}: {t.data.size} elements, expected {n}")


@dataclass
class CoreInputs:
    heads: int
    rows: int
    q: Tensor
    k: Tensor
    v: Tensor
    g: Tensor
    beta: Tensor
    state: np.ndarray  # the reference model's layout, [H][DK][DV]


def core_inputs(s: Set, lf: LayerFixtures, init: Init) -> CoreInputs:
    """goldens.rs:810-883: post-conv q, k (not normalised), v, per-channel log decay, beta, and the state the rows
    start from (the set's own, else the layer's prefill set's final state, else zero)."""
    q, k, v = _tensor(s, lf, Role.Q), _tensor(s, lf, Role.K), _tensor(s, lf, Role.V)
    g, beta = _tensor(s, lf, Role.LogDecay), _tensor(s, lf, Role.Beta)
    if beta.data.size == 0 or q.data.size != beta.data.size * DK:
        raise GoldenError("shape", f"{q.name} and {beta.name} disagree on T * H")
    th = beta.data.size
    if len(beta.shape) >= 2:
        heads = beta.shape[-1]
    elif len(q.shape) >= 2 and q.shape[-1] == DK:
        heads = q.shape[-2]
    else:
        raise GoldenError("shape", f"{q.name}: cannot tell the number of heads")
    if heads == 0 or th % heads != 0:
        raise GoldenError("shape", f"{q.name}: {heads} heads do not divide T * H = {th}")
    for x in (k, g):
        _expect_len(x, th * DK)
    _expect_len(v, th * DV)
    n_state = heads * DK * DV
    si = _optional(s, lf, Role.StateIn)
    if si is not None:
        _expect_len(si, n_state)
        state = si.data
    elif init.state is not None:
        if init.state.size != n_state:
            raise GoldenError("shape", f"initial state: {init.state.size} elements, expected {n_state}")
        state = init.state
    else:
        state = np.zeros(n_state, np.float32)
    return CoreInputs(heads, th // heads, q, k, v, g, beta, np.ascontiguousarray(state, np.float32))


def _is_recurrent(s: Set, lf: LayerFixtures, rows: int) -> bool:
    p = _optional(s, lf, Role.Path)
    return bool((p.data == 1.0).all()) if p is not None else rows == 1


def _transpose_state(x: np.ndarray, heads: int, a: int, b: int) -> np.ndarray:
    """[H][a][b] -> [H][b][a] (the reference model keeps [H][DK][DV], the kernels [H][DV][DK]; cpu.rs:531-547)."""
    return np.ascontiguousarray(x.reshape(heads, a, b).transpose(0, 2, 1)).reshape(-1)


def check_core(s: Set, lf: LayerFixtures, init: Init) -> list:
    """The set's rows through glm53f_kda_core_decode_batch on the GPU (q and k normalised in the kernel, FP32 state),
    row by row when the set holds per-row states: core output, final state and per-row states of the listed heads
    against the fixtures, with the reference's tolerance tiers (goldens.rs:885-955)."""
    import torch

    from . import core

    c = core_inputs(s, lf, init)
    out_ref = _tensor(s, lf, Role.CoreOut)
    _expect_len(out_ref, c.rows * c.heads * DV)
    steps, step_heads = _optional(s, lf, Role.StateSteps), s.state_heads()
    dev = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).cuda() if dt is None else torch.from_numpy(np.ascontiguousarray(a).view(dt)).cuda()
    q, k, v = (dev(_f32_to_bf16(t.data), np.int16) for t in (c.q, c.k, c.v))
    g, beta = dev(c.g.data), dev(c.beta.data)
    state = dev(_transpose_state(c.state, c.heads, DK, DV))
    out = torch.zeros(c.rows * c.heads * DV, dtype=torch.int16, device="cuda")
    off = torch.zeros(1, dtype=torch.int64, device="cuda")
    per_step = []
    if steps is not None and step_heads is not None:
        cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
        w = c.heads * DK
        for r in range(c.rows):
            core.decode_batch(c.heads, 1, cu, q[r * w:(r + 1) * w], k[r * w:(r + 1) * w], v[r * w:(r + 1) * w], g[r * w:(r + 1) * w],
                              beta[r * c.heads:(r + 1) * c.heads], state, off, flags=core.L2NORM, out=out[r * w:(r + 1) * w])
            now = _transpose_state(state.cpu().numpy(), c.heads, DV, DK).reshape(c.heads, DK * DV)
            per_step.append(now[step_heads].reshape(-1))
    else:
        cu = torch.tensor([0, c.rows], dtype=torch.int32, device="cuda")
        core.decode_batch(c.heads, c.rows, cu, q, k, v, g, beta, state, off, flags=core.L2NORM, out=out)
    torch.cuda.synchronize()
    if core.device_status() != 0:
        raise RuntimeError(f"device status {core.device_status()}")
    rec = _is_recurrent(s, lf, c.rows)
    tol = tolerance(out_ref.dtype, rec)
    label = lambda what: f"layer {lf.layer} {what} ({c.rows} rows, {'recurrent' if rec else 'chunked'} path)"
    y = _bf16_to_f32(out.cpu().numpy().view(np.uint16))  # the kernel's output is bf16, as the model's activations are
    results = [Comparison.compare(label("core output"), y, out_ref.data, tol)]
    so = _optional(s, lf, Role.StateOut)
    if so is not None:
        _expect_len(so, c.heads * DK * DV)
        results.append(Comparison.compare(label("state after the rows"), _transpose_state(state.cpu().numpy(), c.heads, DV, DK), so.data, tol))
    if per_step:
        _expect_len(steps, c.rows * len(step_heads) * DK * DV)
        results.append(Comparison.compare(label(f"per-row states of heads {step_heads}"), np.concatenate(per_step), steps.data, tol))
    return results


CORE_ROLES = (Role.Q, Role.K, Role.V, Role.LogDecay, Role.Beta, Role.CoreOut)  # goldens.rs:1244


def write_set(directory: str, tensors, notes=None) -> None:
    """Writes a set: tensors = [(name, DType.F32 | DType.BF16 | DType.I32, shape, values)] (goldens.rs:1276-1310)."""
    os.makedirs(directory, exist_ok=True)
    members = {}
    for name, dtype, shape, values in tensors:
        values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        if values.size != int(np.prod(shape, dtype=np.int64)):
            raise ValueError(f"{name}: shape")
        if dtype is DType.F32:
            data = values.astype("<f4").tobytes()
        elif dtype is DType.BF16:
            data = _f32_to_bf16(values).astype("<u2").tobytes()
        elif dtype is DType.I32:
            data = values.astype("<i4").tobytes()
        else:
            raise ValueError("write_set writes f32, bf16 and i32")
        file = f"{name}.bin"
        with open(os.path.join(directory, file), "wb") as f:
            f.write(data)
        members[name] = {"file": file, "dtype": dtype.manifest_name(), "shape": [int(d) for d in shape], "sha256": hashlib.sha256(data).hexdigest()}
    with open(os.path.join(directory, "manifest.json"), "w") as f:
        json.dump({"tensors": members, "notes": notes}, f, indent=1)
