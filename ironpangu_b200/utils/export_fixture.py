"""Fixtures for qualifying one kernel or one loader outside the engine; nothing here executes a model.

    python -m ironpangu_b200.utils.export_fixture tensor    CHECKPOINT_DIR NAME OUT.bin           # one checkpoint tensor, with header
    python -m ironpangu_b200.utils.export_fixture load-plan BUNDLE_DIR RANK OUT.json              # the rank's init plan, loads resolved
    python -m ironpangu_b200.utils.export_fixture linear    BUNDLE_DIR CHECKPOINT_DIR RANK PARAM OUT.bin [--rows 4] [--seed 0]
    python -m ironpangu_b200.utils.export_fixture moe       BUNDLE_DIR CHECKPOINT_DIR RANK LAYER OUT.bin [--rows 2] [--seed 0]

File layout (little endian): magic ``IFFIXT01``, u32 count, then per array: u32 name length, name, u32 dtype (0 f32, 1 bf16,
2 i32), u32 rank, u64 dims..., u64 byte length, bytes. ``linear``: the rank's shard of ``PARAM`` as the init plan loads it,
random bf16 input rows and the f32-accumulated, bf16-rounded product. ``moe``: router weight, the rank's expert stacks, input
rows, the routing (ids, weights) and the rank's partial output computed in f32. ``read_fixture`` reads a file back.
Tensors above 256 MiB are refused. Reference: crates/inferfabric-cli/examples/export_openpangu_{tensor,load_plan,linear,moe}.rs."""
from __future__ import annotations

import argparse
import json
import struct
import sys
from pathlib import Path
from typing import Dict

import numpy as np
import torch

LIMIT = 256 << 20
_DT = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}
_BACK = {0: torch.float32, 1: torch.bfloat16, 2: torch.int32}


def write_fixture(path: str, arrays: Dict[str, torch.Tensor]) -> None:
    out = bytearray(b"IFFIXT01") + struct.pack("<I", len(arrays))
    for name, t in arrays.items():
        t = t.contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes()
        if len(raw) > LIMIT:
            raise ValueError(f"{name}: {len(raw)} bytes exceed the 256 MiB fixture limit")
        nb = name.encode()
        out += struct.pack("<I", len(nb)) + nb + struct.pack("<II", _DT[t.dtype], t.dim())
        out += b"".join(struct.pack("<Q", d) for d in t.shape) + struct.pack("<Q", len(raw)) + raw
    tmp = Path(str(path) + ".tmp")
    tmp.write_bytes(bytes(out))
    tmp.rename(path)


def read_fixture(path: str) -> Dict[str, torch.Tensor]:
    b = Path(path).read_bytes()
    if b[:8] != b"IFFIXT01":
        raise ValueError("not a fixture file")
    (n,), o, out = struct.unpack_from("<I", b, 8), 12, {}
    for _ in range(n):
        (ln,) = struct.unpack_from("<I", b, o); o += 4
        name = b[o:o + ln].decode(); o += ln
        dt, rank = struct.unpack_from("<II", b, o); o += 8
        dims = struct.unpack_from(f"<{rank}Q", b, o); o += 8 * rank
        (nbytes,) = struct.unpack_from("<Q", b, o); o += 8
        out[name] = torch.frombuffer(bytearray(b[o:o + nbytes]), dtype=torch.uint8).view(_BACK[dt]).view(*dims); o += nbytes
    return out


def _params(bundle: str, checkpoint: str, rank: int, only=None) -> Dict[str, torch.Tensor]:
    from ..runtime.plan_engine import SafetensorsDir, load_parameters

    plan = json.loads((Path(bundle) / f"rank-{rank}.init.json").read_text())
    if only is not None:
        keep = {p["id"] for p in plan["parameters"] if only(p["name"])}
        if not keep:
            raise KeyError("the init plan has no such parameter")
        plan = dict(plan, parameters=[p for p in plan["parameters"] if p["id"] in keep], loads=[l for l in plan["loads"] if l["dest"] in keep])
    return load_parameters(plan, SafetensorsDir(checkpoint), "cpu")


def export_tensor(checkpoint: str, name: str, out: str) -> None:
    from ..runtime.plan_engine import SafetensorsDir

    ck = SafetensorsDir(checkpoint)
    key = name if name in ck.tensors else name + ".weight"
    mm, off, n, dtype, shape = ck.tensors[key]
    if n > LIMIT:
        raise ValueError("tensor exceeds 256 MiB")
    dt = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}[dtype]
    write_fixture(out, {key: torch.frombuffer(bytearray(mm[off:off + n]), dtype=torch.uint8).view(dt).view(*shape)})


def export_load_plan(bundle: str, rank: int, out: str) -> None:
    plan = json.loads((Path(bundle) / f"rank-{rank}.init.json").read_text())
    names = {p["id"]: p["name"] for p in plan["parameters"]}
    doc = {"format": "ifab.load-plan-fixture.v1", "rank": rank, "device_bytes": plan.get("device_bytes"),
           "parameters": plan["parameters"], "loads": [dict(l, parameter=names[l["dest"]]) for l in plan["loads"]]}
    Path(out).write_text(json.dumps(doc, indent=1) + "\n")


def export_linear(bundle: str, checkpoint: str, rank: int, param: str, out: str, rows: int, seed: int) -> None:
    w = _params(bundle, checkpoint, rank, only=lambda n: n == param)[param]
    if w.dim() != 2:
        raise ValueError(f"{param} is not a matrix")
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, w.shape[1], generator=g).to(torch.bfloat16)
    y = (x.float() @ w.float().T).to(torch.bfloat16)
    write_fixture(out, {"weight": w, "input": x, "expected": y})


def export_moe(bundle: str, checkpoint: str, rank: int, layer: int, out: str, rows: int, seed: int) -> None:
    tag = f".layers.{layer}.mlp."
    P = _params(bundle, checkpoint, rank, only=lambda n: tag in n)
    pick = lambda frag: next(v for k, v in P.items() if frag in k)
    router, gu, down = pick("mlp.gate"), pick("experts.{expert}.gate_proj"), pick("experts.{expert}.down_proj")
    program = json.loads((Path(bundle) / "device-program.json").read_text())
    r = next(i for i in program["instructions"] if i["op"] == "router_topk" and tag in i["attrs"]["weight"] + ".")
    topk, E, el = int(r["attrs"]["topk"]), router.shape[0], gu.shape[0]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, router.shape[1], generator=g).to(torch.bfloat16)
    logits = x.float() @ router.float().T
    score = torch.softmax(logits, -1) if r["attrs"]["scoring"] == "softmax" else torch.sigmoid(logits)
    wts, ids = score.topk(topk, -1)
    wts = wts / wts.sum(-1, keepdim=True) * float(r["attrs"]["scale"])
    F = gu.shape[1] // 2
    y = torch.zeros(rows, down.shape[1])
    for t in range(rows):
        for k in range(topk):
            e = int(ids[t, k]) - rank * el
            if 0 <= e < el:
                h = x[t].float() @ gu[e].float().T
                a = (torch.nn.functional.silu(h[:F]) * h[F:]).to(torch.bfloat16).float()
                y[t] += wts[t, k] * (a @ down[e].float().T)
    write_fixture(out, {"router": router, "gate_up": gu, "down": down, "input": x, "route_ids": ids.to(torch.int32), "route_weights": wts,
                        "expected_partial": y})


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="verb", required=True)
    t = sub.add_parser("tensor"); t.add_argument("checkpoint"); t.add_argument("name"); t.add_argument("out")
    l = sub.add_parser("load-plan"); l.add_argument("bundle"); l.add_argument("rank", type=int); l.add_argument("out")
    for verb, what in (("linear", "param"), ("moe", "layer")):
        p = sub.add_parser(verb)
        p.add_argument("bundle"); p.add_argument("checkpoint"); p.add_argument("rank", type=int)
        p.add_argument(what, type=int if what == "layer" else str); p.add_argument("out")
        p.add_argument("--rows", type=int, default=4 if verb == "linear" else 2); p.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.verb == "tensor":
        export_tensor(a.checkpoint, a.name, a.out)
    elif a.verb == "load-plan":
        export_load_plan(a.bundle, a.rank, a.out)
    elif a.verb == "linear":
        export_linear(a.bundle, a.checkpoint, a.rank, a.param, a.out, a.rows, a.seed)
    else:
        export_moe(a.bundle, a.checkpoint, a.rank, a.layer, a.out, a.rows, a.seed)
    return 0


if __name__ == "__main__":
    sys.exit(main())
