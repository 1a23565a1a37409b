#!/usr/bin/env python
"""Times the reference project's own sm_100 kernels on this GPU: the fused norm + A-plane
kernel, the chained gate_up GEMM and the rank-split down GEMM of one MLP layer, through the
reference's own `build_chain` plans (lcgemm/seams/__init__.py:19-38 of that project).

Runs in a process of its own because the reference package and this repository's package
share the name `lcgemm`: here only the unmodified install under baseline/_ref is importable
(`pip install --no-deps --target baseline/_ref <reference tree>`; git-ignored).  One GPU only:
the reference's kernels pass a cluster mask to their TMA copies.  Prints one JSON line;
a stage that fails to import, JIT-compile or run is reported with its error text instead of a
time, and nothing is retried.

    python baseline/ref_kernels.py TOKENS STEPS WARMUP [DUMP.pt|-] [HIDDEN INTER]

With DUMP.pt the kernels' outputs on the seeded inputs (residual stream, A planes, Z, the
consumer's planes, the layer output) are saved there with torch.save, so that the caller can
hold its own kernels' bits against them.  The inputs are bench.py's `make_layer_tensors`
(seed 0) restated: x and the norm weight from one generator, the weights from a second.
"""
import json
import statistics
import sys
import traceback
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def _short(exc: BaseException) -> str:
    text = "".join(traceback.format_exception_only(type(exc), exc)).strip()
    return text[-600:]


def main() -> None:
    tokens = int(sys.argv[1]) if len(sys.argv) > 1 else 2048
    steps = int(sys.argv[2]) if len(sys.argv) > 2 else 20
    warmup = int(sys.argv[3]) if len(sys.argv) > 3 else 3
    dump = sys.argv[4] if len(sys.argv) > 4 and sys.argv[4] != "-" else None
    hidden = int(sys.argv[5]) if len(sys.argv) > 5 else 5120
    inter = int(sys.argv[6]) if len(sys.argv) > 6 else 17408
    eps = 1e-6
    out = {"ref_kernels_child": True, "tokens": tokens, "hidden": hidden, "inter": inter,
           "steps": steps, "warmup": warmup, "stages": {}, "versions": {}}
    if not (REF / "lcgemm").is_dir():
        out["unavailable"] = "baseline/_ref holds no install of the reference"
        print(json.dumps(out))
        return
    sys.path.insert(0, str(REF))
    try:
        import torch

        import cutlass
        import lcgemm
        from lcgemm.seams import build_chain

        assert str(REF) in str(Path(lcgemm.__file__).resolve()), lcgemm.__file__
        out["versions"] = {"torch": torch.__version__,
                           "nvidia-cutlass-dsl": getattr(cutlass, "__version__", "?")}
    except BaseException as exc:            # noqa: BLE001 - report, never retry
        out["unavailable"] = "import failed: " + _short(exc)
        print(json.dumps(out))
        return

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16
    x = torch.randn((tokens, hidden), generator=g, device=dev).to(bf)
    nw = (torch.randn((hidden,), generator=g, device=dev) * 0.01).to(bf)
    gw = torch.Generator(device=dev).manual_seed(1000)
    wgu = (torch.randn((2 * inter, hidden), generator=gw, device=dev) * 0.02).to(bf)
    wd = (torch.randn((hidden, inter), generator=gw, device=dev) * 0.02).to(bf)
    zero = torch.zeros_like(x)
    flush = torch.empty(256 << 20, dtype=torch.int8, device=dev)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ms = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        return {"mean_us": statistics.mean(ms) * 1e3, "median_us": statistics.median(ms) * 1e3,
                "min_us": min(ms) * 1e3}

    try:
        gate, down = build_chain((tokens, hidden, 2 * inter), (tokens, inter, hidden))
        gate_bw = gate.prepare_weight(wgu)
        down_bw = down.prepare_weight(wd)
        torch.cuda.synchronize()
    except BaseException as exc:            # noqa: BLE001
        out["unavailable"] = "build_chain / prepare_weight failed: " + _short(exc)
        print(json.dumps(out))
        return

    state = {}
    stages = (
        ("norm_planes", lambda: state.__setitem__("a", gate.a_planes(x, zero, nw, eps))),
        ("gate_up", lambda: gate.gemm(state["a"], gate_bw)),
        ("down", lambda: down.gemm(down.a_planes(), down_bw)),
    )
    for name, fn in stages:
        try:
            fn()                             # first call JIT-compiles
            torch.cuda.synchronize()
            out["stages"][name] = timed(fn)
        except BaseException as exc:        # noqa: BLE001
            out["stages"][name] = {"unavailable": _short(exc)}
            break                            # later stages consume this one's output
    if dump and all("mean_us" in out["stages"].get(k, {}) for k in ("norm_planes", "gate_up", "down")):
        try:
            gate.a_planes(x, zero, nw, eps)
            gate.gemm(gate.a, gate_bw)
            down.gemm(down.a_planes(), down_bw)
            torch.cuda.synchronize()
            torch.save({"residual_out": gate.residual_out.cpu(), "a_planes": gate.a.cpu(), "z": gate.c.cpu(),
                        "planes": gate.planes.cpu(), "out": down.c.cpu(),
                        "gate_bw": gate_bw[:4096].cpu(), "down_bw": down_bw[:4096].cpu()}, dump)
            out["dump"] = dump
        except BaseException as exc:        # noqa: BLE001
            out["dump"] = "failed: " + _short(exc)
    try:
        out["describe"] = {"gate_up": gate.describe(), "down": down.describe()}
    except BaseException:                   # noqa: BLE001
        pass
    # the reference's own functional layer beside its kernels' output, as a sanity figure
    try:
        if "down" in out["stages"] and "mean_us" in out["stages"]["down"]:
            rows = slice(0, 256)
            h = x[rows].float()
            y = h * torch.rsqrt(h.square().mean(-1, keepdim=True) + eps) * (nw.float() + 1.0)
            z = torch.nn.functional.linear(y.to(bf), wgu)
            gate_z, up_z = z.chunk(2, dim=-1)
            want = torch.nn.functional.linear(torch.nn.functional.silu(gate_z.float()).to(bf) * up_z, wd)
            got = down.c[rows]
            out["rel_fro_vs_functional"] = float(((got.float() - want.float()).norm() / want.float().norm()).item())
    except BaseException as exc:            # noqa: BLE001
        out["rel_fro_vs_functional"] = "failed: " + _short(exc)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
