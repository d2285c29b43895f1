"""Calibrated 3-bit decode copies for a whole model: capture, fit, write, attach.

    python -m hibana_b200.weights.calibrate_model --target dense-27b --inputs samples.json --output DIR
    python -m hibana_b200 serve dense-27b --w3 --w3-checkpoint DIR

1. Capture. The model is built (or loaded) with its projections in bf16, an `Executor` prefills the calibration
   samples, and every `Linear` call adds x^T x of the rows it sees to its projection's covariance (`Covariances`
   patches `Linear.__call__` for the length of the capture). These are the activations of the serving path: the
   norms, the attention and the recurrences in front of a projection are the real kernels.
2. Fit. Every projection whose shape the 3-bit kernel tiles (K a multiple of 64) is fitted with GPTQ onto the
   kernel's format (`w3_calibrate.gptq_int3g64`: asymmetric 3-bit integers, groups of 64, the rounding error of a
   column pushed onto the columns still to come through the inverse covariance). The report lists the relative
   output error of the fitted copy and of plain round-to-nearest on the captured covariance.
3. Write. One safetensors file per matrix (`codes` packed two per byte, `scale`, `zero`) and a manifest with shapes
   and sha256 digests; `load_directory` checks the digests before it hands a matrix out.
4. Attach. `attach(model, directory)` replaces the uncalibrated decode copies (`Linear.attach_w3`) of the
   projections the directory names; the others keep theirs.
Routed experts are stacked tensors, not `Linear`s: `ExpertCovariances` collects, per expert, the covariance of the
rows routed to it (weighted by the routing weight) for both of its matrices, `fit_experts` runs the same GPTQ per
expert (experts with too few rows keep nearest rounding) and the stacks are written as `<layer>.experts.fc1|fc2`;
`attach` hands them to the layer (`MoeLayer.attach_w3`).
Reference: hibana/weights/flashnext_w3_calibrate.py:1-115, nemotron_w3_calibrate.py, bolt_w3_calibrate.py (one driver
per family there; the capture is the same in all three), hibana/weights/w3_checkpoint.py:57-208 (manifest + sha256).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import time
from pathlib import Path
from typing import Iterable, Optional, Sequence

import torch

from ..models.linear import Linear
from ..ops.nvfp4 import Nvfp4Tensor
from .w3 import Int3G64
from .w3_calibrate import gptq_int3g64

FORMAT = "hibana_b200-int3g64-v1"
MANIFEST = "manifest.json"


class Covariances:
    """x^T x per named projection, accumulated from `Linear` calls while the context is open."""

    def __init__(self, linears: Iterable[Linear], device=None):
        self.names = {id(lin): lin.name for lin in linears if lin.name}
        self.matrices: dict = {}
        self.rows: dict = {}
        self.device = device

    def __enter__(self) -> "Covariances":
        self._original = Linear.__call__
        cov = self

        def call(lin, x, **kw):
            name = cov.names.get(id(lin))
            if name is not None and not isinstance(x, Nvfp4Tensor):
                xf = x.detach().reshape(-1, x.shape[-1]).float()
                if cov.device is not None:
                    xf = xf.to(cov.device)
                h = cov.matrices.get(name)
                if h is None:
                    h = cov.matrices[name] = torch.zeros(xf.shape[1], xf.shape[1], dtype=torch.float32, device=xf.device)
                h.addmm_(xf.t(), xf)
                cov.rows[name] = cov.rows.get(name, 0) + xf.shape[0]
            return cov._original(lin, x, **kw)
        Linear.__call__ = call
        return self

    def __exit__(self, *exc) -> None:
        Linear.__call__ = self._original


def expert_layers(model) -> dict:
    """{name: MoE layer} of the layers whose routed experts are stacked tensors (`l{i}.ffn.experts`)."""
    from ..models.layers import MoeLayer
    out = {}
    for blk in getattr(model, "blocks", []):
        ffn = getattr(blk, "ffn", None)
        if isinstance(ffn, MoeLayer):
            out[ffn.router.name[:-len(".router")] + ".experts"] = ffn
    return out


class ExpertCovariances:
    """Per-expert input covariances of the routed experts, from `moe.experts_forward` calls while the context is
    open: for expert e of a layer, H1[e] = sum g^2 x x^T over the rows routed to it (x the expert's input, g the
    routing weight) and H2[e] the same over h = act(fc1_e x), the input of its second matrix. Rows a token sends to
    an expert it weighs lightly count lightly. Reference: hibana/weights/nemotron_w3_experts.py:17-22."""

    def __init__(self, model):
        self.layers = expert_layers(model)
        self.names = {id(layer.experts): name for name, layer in self.layers.items()}
        self.h1: dict = {}
        self.h2: dict = {}
        self.rows: dict = {}
        self._dense: dict = {}

    def _add(self, name, x, ids, weights, ew, id_base):
        from ..ops.moe import _act
        if name not in self.h1:
            self.h1[name] = torch.zeros(ew.experts, ew.hidden, ew.hidden)
            self.h2[name] = torch.zeros(ew.experts, ew.inter, ew.inter)
            self.rows[name] = torch.zeros(ew.experts, dtype=torch.int64)
            self._dense[name] = ew.dense(1).float().cpu()
        xf, idc, wc = x.detach().float().cpu(), ids.detach().cpu().long() - id_base, weights.detach().float().cpu()
        for e in idc.unique().tolist():
            if e < 0 or e >= ew.experts:
                continue
            tok, slot = (idc == e).nonzero(as_tuple=True)
            g = wc[tok, slot][:, None]
            xe = xf[tok]
            self.h1[name][e].addmm_((xe * g).t(), xe * g)
            h = _act(xe @ self._dense[name][e].t(), ew.act).to(torch.bfloat16).float()
            self.h2[name][e].addmm_((h * g).t(), h * g)
            self.rows[name][e] += tok.numel()

    def __enter__(self) -> "ExpertCovariances":
        from ..ops import moe as moe_ops
        self._original = moe_ops.experts_forward
        cov = self

        def forward(x, ids, weights, ew, **kw):
            name = cov.names.get(id(ew))
            if name is not None:
                cov._add(name, x, ids, weights, ew, kw.get("id_base", 0))
            return cov._original(x, ids, weights, ew, **kw)
        moe_ops.experts_forward = forward
        return self

    def __exit__(self, *exc) -> None:
        from ..ops import moe as moe_ops
        moe_ops.experts_forward = self._original


def fit_experts(model, ecov: ExpertCovariances, *, min_rows: int = 32, log=None) -> tuple[dict, list]:
    """GPTQ every routed expert that saw at least `min_rows` rows on its own covariances; the others keep nearest
    rounding. Returns ({"<layer>.experts.fc1" / ".fc2": Int3G64 over all experts' rows}, report rows)."""
    fitted, report = {}, []
    for name, layer in ecov.layers.items():
        if name not in ecov.h1:
            continue
        ew = layer.experts
        if ew.n1 % 128 or ew.fc2_rows % 128 or ew.hidden % 64 or ew.inter % 64:
            continue
        t0 = time.perf_counter()
        row = {"name": name, "experts": ew.experts, "calibrated": 0}
        for which, hs in ((1, ecov.h1[name]), (2, ecov.h2[name])):
            dense = ew.dense(which).float().cpu()
            parts, err_g, err_n, fitted_n = [], 0.0, 0.0, 0
            for e in range(ew.experts):
                w = dense[e]
                plain = Int3G64.quantize(w)
                if int(ecov.rows[name][e]) >= min_rows:
                    q = gptq_int3g64(w, hs[e])
                    err_g += relative_error(w, q.dequantize(), hs[e])
                    err_n += relative_error(w, plain.dequantize(), hs[e])
                    fitted_n += 1
                else:
                    q = plain
                parts.append(q)
            fitted[f"{name}.fc{which}"] = Int3G64(torch.cat([q.codes for q in parts]),
                                                  torch.cat([q.scale for q in parts]),
                                                  torch.cat([q.zero for q in parts]))
            row[f"fc{which}_error_gptq"] = round(err_g / max(fitted_n, 1), 5)
            row[f"fc{which}_error_nearest"] = round(err_n / max(fitted_n, 1), 5)
            row["calibrated"] = fitted_n
        row["seconds"] = round(time.perf_counter() - t0, 2)
        report.append(row)
        if log is not None:
            log(json.dumps(row))
    return fitted, report


def to_bf16(model) -> None:
    """Puts every projection of `model` in bf16 in place (a capture model: activations reach the projections
    unquantised, so the covariances are those of the bf16 trunk)."""
    for lin in model.linears():
        if lin.fmt == "bf16" or not isinstance(lin, Linear):
            continue
        dev = lin.wq.q.device
        lin.weight = lin.dequantized().to(torch.bfloat16).to(dev).contiguous()
        lin.fmt, lin.wq = "bf16", None


def capture(model, samples: Sequence[Sequence[int]], *, max_batch: int = 4, chunk: int = 0) -> Covariances:
    """Prefills `samples` (token id lists) through an Executor and returns the covariances of every projection."""
    from ..engine.executor import Executor
    from ..engine.request import SamplingParams
    longest = max(len(s) for s in samples)
    ex = Executor(model, max_batch=max_batch, max_ctx=longest + 16, use_graphs=False, radix_cache=False)
    cov = Covariances(model.linears())
    cov.experts = ExpertCovariances(model)        # the routed experts' own covariances, from the same prefills
    with cov, cov.experts:
        for i in range(0, len(samples), max_batch):
            ex.generate_batch([list(s) for s in samples[i:i + max_batch]], SamplingParams(max_tokens=1))
    return cov


def relative_error(w: torch.Tensor, wq: torch.Tensor, h: torch.Tensor) -> float:
    """||X w^T - X wq^T|| / ||X w^T|| from the covariance alone: tr(D H D^T) / tr(W H W^T) with D = w - wq."""
    d = (w.float() - wq.float()).to(h.device)
    wf = w.float().to(h.device)
    num = ((d @ h) * d).sum()
    den = ((wf @ h) * wf).sum().clamp_min(1e-30)
    return float(torch.sqrt(num / den))


def fit(model, cov: Covariances, *, log=None) -> tuple[dict, list]:
    """GPTQ every captured projection. Returns ({name: Int3G64}, report rows)."""
    fitted, report = {}, []
    for lin in model.linears():
        h = cov.matrices.get(getattr(lin, "name", ""))
        if h is None or lin.in_features % 64:
            continue
        w = lin.dequantized().to(h.device)
        t0 = time.perf_counter()
        q = gptq_int3g64(w, h)
        plain = Int3G64.quantize(w)
        row = {"name": lin.name, "shape": [lin.out_features, lin.in_features], "rows": cov.rows[lin.name],
               "error_gptq": round(relative_error(w, q.dequantize(), h), 5),
               "error_nearest": round(relative_error(w, plain.dequantize(), h), 5),
               "seconds": round(time.perf_counter() - t0, 2)}
        fitted[lin.name] = q
        report.append(row)
        if log is not None:
            log(json.dumps(row))
    return fitted, report


def _sha256(path: Path) -> str:
    dig = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 22), b""):
            dig.update(block)
    return dig.hexdigest()


def write_directory(directory, fitted: dict, *, target: str = "", report: Optional[list] = None) -> Path:
    from safetensors.torch import save_file
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    manifest = {"format": FORMAT, "target": target, "weights": {}, "report": report or []}
    for i, (name, q) in enumerate(sorted(fitted.items())):
        codes = q.codes.cpu()
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
        fname = f"int3-{i:05d}.safetensors"
        save_file({"codes": packed, "scale": q.scale.cpu().contiguous(), "zero": q.zero.cpu().contiguous()},
                  str(d / fname))
        manifest["weights"][name] = {"file": fname, "sha256": _sha256(d / fname), "out_features": codes.shape[0],
                                     "in_features": codes.shape[1]}
    (d / MANIFEST).write_text(json.dumps(manifest, indent=1))
    return d


def load_directory(directory, names: Optional[Iterable[str]] = None, verify: bool = True) -> dict:
    """{name: Int3G64} of the matrices in `directory` (all, or `names`); a digest mismatch raises."""
    from safetensors.torch import load_file
    d = Path(directory)
    manifest = json.loads((d / MANIFEST).read_text())
    if manifest.get("format") != FORMAT:
        raise ValueError(f"{d}: not a {FORMAT} directory")
    out = {}
    for name, entry in manifest["weights"].items():
        if names is not None and name not in names:
            continue
        path = d / entry["file"]
        if verify and _sha256(path) != entry["sha256"]:
            raise ValueError(f"{path}: sha256 differs from the manifest")
        t = load_file(str(path))
        packed = t["codes"]
        codes = torch.stack((packed & 7, packed >> 4), dim=-1).reshape(packed.shape[0], -1)
        if tuple(codes.shape) != (entry["out_features"], entry["in_features"]):
            raise ValueError(f"{name}: shape differs from the manifest")
        out[name] = Int3G64(codes.contiguous(), t["scale"], t["zero"])
    return out


def attach(model, directory, *, strict: bool = False) -> int:
    """Gives the projections `directory` names their calibrated decode copies. Returns how many were attached;
    `strict` raises when the directory names a projection the model does not have (or of another shape)."""
    from ..ops.w3gemm import W3Linear
    by_name = {lin.name: lin for lin in model.linears() if getattr(lin, "name", "")}
    fitted = load_directory(directory)
    moes = expert_layers(model)
    stacks = {f"{name}.fc{w}" for name in moes for w in (1, 2)}
    unknown = sorted(set(fitted) - set(by_name) - stacks)
    if unknown and strict:
        raise ValueError(f"calibrated names not in this model: {unknown[:4]}")
    n = 0
    for name, q in fitted.items():
        lin = by_name.get(name)
        if lin is None:
            continue
        if q.shape != (lin.out_features, lin.in_features):
            if strict:
                raise ValueError(f"{name}: calibrated shape {q.shape} != {(lin.out_features, lin.in_features)}")
            continue
        dev = lin.weight.device if lin.weight is not None else lin.wq.q.device
        lin.w3 = W3Linear(q, dev, name=name + ".w3", keep_codes=dev.type != "cuda")
        n += 1
    for name, layer in moes.items():
        q1, q2 = fitted.get(f"{name}.fc1"), fitted.get(f"{name}.fc2")
        if q1 is None or q2 is None:
            continue
        ew = layer.experts
        if q1.shape != (ew.experts * ew.n1, ew.hidden) or q2.shape != (ew.experts * ew.fc2_rows, ew.inter):
            if strict:
                raise ValueError(f"{name}: calibrated expert stacks {q1.shape} / {q2.shape} do not match the layer")
            continue
        layer.attach_w3(q1, q2)
        n += 1
    return n


def load_samples(path) -> list:
    """{"samples": [[token id, ...], ...]} (or a bare list of lists)."""
    data = json.loads(Path(path).read_text())
    return data["samples"] if isinstance(data, dict) else data


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--target", required=True)
    ap.add_argument("--weights", default="", help="checkpoint directory (default: random-init weights of the target)")
    ap.add_argument("--inputs", required=True, help="calibration samples: JSON token id lists")
    ap.add_argument("--output", required=True)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--layers", type=int, default=0, help="first N blocks only (smoke runs)")
    ap.add_argument("--max-batch", type=int, default=4)
    ap.add_argument("--min-expert-rows", type=int, default=32,
                    help="routed experts that saw fewer calibration rows keep nearest rounding")
    args = ap.parse_args(argv)
    from ..engine.llm import build_model
    from ..target import get_target, scaled
    full = get_target(args.target)
    t = scaled(full, layers=args.layers) if args.layers else full
    # random-init targets are built in bf16 from the same seed (the weights the served NVFP4 copies were rounded
    # from); a checkpoint's projections are expanded to bf16 after loading
    model = build_model(t, args.device, weights=args.weights) if args.weights else \
        build_model(scaled(t, weight_format="bf16"), args.device)
    to_bf16(model)
    cov = capture(model, load_samples(args.inputs), max_batch=args.max_batch)
    fitted, report = fit(model, cov, log=print)
    if cov.experts.h1:
        efit, ereport = fit_experts(model, cov.experts, min_rows=args.min_expert_rows, log=print)
        fitted.update(efit)
        report += ereport
    out = write_directory(args.output, fitted, target=t.name, report=report)
    lins = [r for r in report if "error_gptq" in r]
    print(json.dumps({"directory": str(out), "matrices": len(fitted),
                      "mean_error_gptq": round(sum(r["error_gptq"] for r in lins) / max(len(lins), 1), 5),
                      "mean_error_nearest": round(sum(r["error_nearest"] for r in lins) / max(len(lins), 1), 5),
                      "expert_layers": len(report) - len(lins)}))


if __name__ == "__main__":
    main()
