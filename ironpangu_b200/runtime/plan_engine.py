"""Executor of a compiled bundle on one rank.

``PlanEngine`` reads ``device-program.json`` and this rank's IFINIT01 plan from a bundle directory,
streams the weight slices from the safetensors checkpoint into device parameters (row shards,
strided column shards, local experts, packed pairs - exactly as the plan says) and then runs the
physical instructions by dispatching each one to its sm_100a kernel. The instruction loop is only
walked eagerly for prefill chunks and once during CUDA-graph capture; steady-state decode replays
the captured graph.

Reference counterparts: the init-plan executor (native/src/initialization_plan.cpp:192-278) and the
token dispatcher (native/src/token_dispatch.inc:19-294).
"""
from __future__ import annotations

import json
import math
import mmap
import os
import struct
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

from ..ops import decode as K
from ..ops import hc as HC
from ..parallel.fabric import Fabric

BF16 = torch.bfloat16
_DT = {"bf16": (torch.bfloat16, 2), "f32": (torch.float32, 4), "int8": (torch.int8, 1), "fp8_e4m3": (torch.float8_e4m3fn, 1)}


class SafetensorsDir:
    """Read-only view of every ``*.safetensors`` file of a directory (headers parsed, data mmapped)."""

    def __init__(self, path: str):
        self.tensors: Dict[str, tuple] = {}
        self.files: Dict[str, mmap.mmap] = {}
        self._maps = []
        for f in sorted(Path(path).glob("*.safetensors")):
            fh = open(f, "rb")
            mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps.append((fh, mm))
            self.files[f.name] = mm
            (hlen,) = struct.unpack("<Q", mm[:8])
            hdr = json.loads(mm[8:8 + hlen])
            for name, info in hdr.items():
                if name == "__metadata__":
                    continue
                b, e = info["data_offsets"]
                self.tensors[name] = (mm, 8 + hlen + b, e - b, info["dtype"], info["shape"])

    def bytes_of(self, name: str) -> np.ndarray:
        mm, off, n, _, _ = self.tensors[name]
        return np.frombuffer(mm, dtype=np.uint8, count=n, offset=off)

    def shard_from(self, shard: str, offset: int) -> np.ndarray:
        """The bytes of shard file ``shard`` from absolute file offset ``offset`` to its end."""
        mm = self.files[shard]
        if offset < 0 or offset > len(mm):
            raise ValueError(f"offset {offset} is outside {shard} ({len(mm)} bytes)")
        return np.frombuffer(mm, dtype=np.uint8, count=len(mm) - offset, offset=offset)


def load_parameters(init_plan: dict, ckpt: SafetensorsDir, device, *, staging_bytes: int = 64 << 20, transfers=None) -> Dict[str, torch.Tensor]:
    """Execute one rank's initialization plan: returns ``{parameter name: device tensor}``.

    Bytes travel through ONE staging buffer of ``staging_bytes`` (pinned when the destination is a GPU), so loading a shard of
    any size costs a bounded amount of host memory; strided loads (column shards) are gathered row block by row block into
    the same buffer. Every upload is recorded under the ``parameter_preparation`` role of ``transfers`` (a
    ``runtime.transfers.TransferAudit``) when one is given.
    Reference: bounded staging + verify of the native init executor (crates/inferfabric-native/src/initialization.rs)."""
    from .transfers import TransferAudit

    tr = transfers if transfers is not None else TransferAudit()
    on_gpu = torch.device(device).type == "cuda"
    stage = torch.empty(max(4096, int(staging_bytes)), dtype=torch.uint8)
    if on_gpu:
        stage = stage.pin_memory()
    stage_np = stage.numpy()
    params, cursors, raw = {}, {}, {}
    for p in init_plan["parameters"]:
        dt, eb = _DT[p["dtype"]]
        n = int(np.prod(p["dims"])) * eb
        raw[p["id"]] = torch.empty(n, dtype=torch.uint8, device=device)
        cursors[p["id"]] = 0
    meta = {p["id"]: p for p in init_plan["parameters"]}

    def upload(dest: int, nbytes: int, widen: bool) -> None:
        """``stage[:nbytes]`` -> the next bytes of parameter ``dest`` (bf16 -> f32 widening on the device when asked)."""
        c = cursors[dest]
        with tr.scope("parameter_preparation"):
            if widen:
                tmp = tr.upload(stage[:nbytes], device, non_blocking=False)
                raw[dest][c:c + 2 * nbytes].copy_(tmp.view(torch.bfloat16).to(torch.float32).view(torch.uint8))
                cursors[dest] = c + 2 * nbytes
            else:
                tr.h2d(raw[dest][c:c + nbytes], stage[:nbytes], non_blocking=False)     # the buffer is reused at once
                cursors[dest] = c + nbytes

    for l in init_plan["loads"]:
        # a load names the shard FILE and an absolute offset inside it (the safetensors header included)
        src = ckpt.shard_from(l["shard"], l["offset"])
        dst_dt = meta[l["dest"]]["dtype"]
        widen = l["src_dtype"] == "bf16" and dst_dt == "f32"
        if not widen and l["src_dtype"] != dst_dt:
            raise ValueError(f"no conversion {l['src_dtype']} -> {dst_dt} for {l.get('tensor', l['shard'])}")
        if l["kind"] == "slice":
            if l["bytes"] > src.size:
                raise ValueError(f"load of {l.get('tensor', l['shard'])} runs past the end of {l['shard']}")
            step = stage.numel() // 4 * 4
            for b in range(0, l["bytes"], step):
                n = min(step, l["bytes"] - b)
                stage_np[:n] = src[b:b + n]
                upload(l["dest"], n, widen)
        else:
            rb, sb = l["row_bytes"], l["stride_bytes"]
            rows = l["bytes"] // rb
            if (rows - 1) * sb + rb > src.size:
                raise ValueError(f"strided load of {l.get('tensor', l['shard'])} runs past the end of {l['shard']}")
            if rb > stage.numel():
                raise ValueError(f"a row of {l.get('tensor', l['shard'])} ({rb} bytes) does not fit the staging buffer")
            per = max(1, stage.numel() // rb)
            for r0 in range(0, rows, per):
                nr = min(per, rows - r0)
                view = np.lib.stride_tricks.as_strided(src[r0 * sb:], shape=(nr, rb), strides=(sb, 1))
                stage_np[:nr * rb].reshape(nr, rb)[:] = view
                upload(l["dest"], nr * rb, widen)
    for pid, p in meta.items():
        if cursors[pid] != raw[pid].numel():
            raise ValueError(f"parameter {p['name']} was filled with {cursors[pid]} of {raw[pid].numel()} bytes")
        params[p["name"]] = raw[pid].view(_DT[p["dtype"]][0]).view(*p["dims"])
    return params


def random_parameters(init_plan: dict, device, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random-init tensors for every parameter of one rank's initialization plan, without a checkpoint: each load slice is
    drawn from a generator keyed by (checkpoint tensor name, byte offset, seed), so a replicated tensor is identical on every
    rank and the shards of a split tensor differ. N(0, ``std``); tensors whose name says they are a norm gain get 1 + N(0, ``std``).
    For benchmarks and tests of programs whose checkpoint is too large to write (a bundle compiled without a checkpoint
    records the same loads against a synthetic layout)."""
    meta = {p["id"]: p for p in init_plan["parameters"]}
    raw, cursors = {}, {}
    for p in init_plan["parameters"]:
        dt, _ = _DT[p["dtype"]]
        raw[p["id"]] = torch.empty(int(np.prod(p["dims"])), dtype=dt, device=device)
        cursors[p["id"]] = 0
    gen = torch.Generator(device=device)
    for l in init_plan["loads"]:
        n = l["bytes"] // _DT[l["src_dtype"]][1]
        gen.manual_seed(_fnv1a64(f"{l.get('tensor', l['shard'])}@{l['offset']}#{seed}".encode()) & 0x7FFFFFFFFFFFFFFF)
        piece = torch.empty(n, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
        if "norm" in l.get("tensor", ""):
            piece += 1.0
        c = cursors[l["dest"]]
        raw[l["dest"]][c:c + n].copy_(piece)
        cursors[l["dest"]] = c + n
    out = {}
    for pid, p in meta.items():
        if cursors[pid] != raw[pid].numel():
            raise ValueError(f"parameter {p['name']} was filled with {cursors[pid]} of {raw[pid].numel()} elements")
        out[p["name"]] = raw[pid].view(*p["dims"])
    return out


def _fnv1a64(data: bytes) -> int:
    h = 0xcbf29ce484222325
    for b in data:
        h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h


class FrozenArena:
    """The activation arena a bundle was compiled with (``arena-rank-N.txt``, IFARENA2, and ``workspace-rank-N.txt``,
    IFWORKSPACE1): ONE device block, every instruction result a view at the offset the compiler planned for it.

    Rules (the reference's frozen arena: native/include/frozen_arena.h:26-54, native/src/prepared_execution.h:189-239):
    the files' program fingerprint must be that of the bundle's ``execution.bin`` (a plan made for another program is
    refused), the plan must cover at least as many query rows as the engine runs, a lease must fit its slot exactly or
    leave room (never grow it), every instruction leases at most once, and nothing is allocated after construction."""

    def __init__(self, bundle: Path, rank: int, rows: int, device):
        text = (bundle / f"arena-rank-{rank}.txt").read_text().split("\n")
        head = text[0].split()
        if len(head) != 5 or head[0] != "IFARENA2":
            raise ValueError("arena file is not IFARENA2")
        want = _fnv1a64((bundle / "execution.bin").read_bytes())
        if int(head[1], 16) != want:
            raise ValueError(f"arena was planned for another program (fingerprint {head[1]}, this bundle's program has {want:016x})")
        self.bytes, n = int(head[3]), int(head[4])
        sizes = [tuple(int(x) for x in text[1 + i].split()) for i in range(n)]
        if text[1 + n].strip() != "pool":
            raise ValueError("arena file lacks its pool section")
        owners = [tuple(int(x) for x in text[2 + n + i].split()) for i in range(n)]
        tokens_line = text[2 + 2 * n].split()
        self.tokens = int(tokens_line[1]) if len(tokens_line) == 2 and tokens_line[0] == "tokens" else 1
        if self.tokens < rows:
            raise ValueError(f"arena was planned for {self.tokens} query rows, the engine runs {rows}: compile the bundle with "
                             f"prefill_tokens >= {rows}")
        self.slots: Dict[int, tuple] = {}
        self.live: Dict[int, tuple] = {}          # instruction -> (first, last) instruction index during which its slot is its own
        for (off, size), (ins, first, last) in zip(sizes, owners):
            if off % 512 or size % 512 or off + size > self.bytes:
                raise ValueError(f"arena slot of instruction {ins} is misaligned or outside the arena")
            self.slots[ins] = (off, size)
            self.live[ins] = (first, last)
        ws = (bundle / f"workspace-rank-{rank}.txt").read_text().split()
        if len(ws) != 4 or ws[0] != "IFWORKSPACE1" or int(ws[1], 16) != want:
            raise ValueError("workspace file does not belong to this bundle's program")
        self.workspace_bytes = int(ws[3])
        self.block = torch.zeros(self.bytes + self.workspace_bytes, dtype=torch.uint8, device=device)   # the one allocation
        self.leased: Dict[int, int] = {}

    def lease(self, instruction: int, nbytes: int) -> torch.Tensor:
        """The planned slot of ``instruction`` as a byte tensor of ``nbytes``; raises when there is no slot, when it is smaller
        than asked (the plan and the engine disagree on a shape) or when it was leased before."""
        if instruction not in self.slots:
            raise RuntimeError(f"the arena has no slot for instruction {instruction}")
        if instruction in self.leased:
            raise RuntimeError(f"instruction {instruction} leased its arena slot twice")
        off, size = self.slots[instruction]
        if nbytes > size:
            raise RuntimeError(f"instruction {instruction} needs {nbytes} bytes, its arena slot holds {size}")
        self.leased[instruction] = nbytes
        return self.block[off:off + nbytes]

    def workspace(self, nbytes: int) -> torch.Tensor:
        if nbytes > self.workspace_bytes:
            raise RuntimeError(f"a kernel needs {nbytes} bytes of workspace, the plan froze {self.workspace_bytes}")
        return self.block[self.bytes:self.bytes + nbytes]


class PlanEngine:
    """Runs a bundle's physical program for up to ``max_tokens`` (<= 8) query rows per step. Activations live in the bundle's
    frozen arena (one device block laid out by the compiler); sequence state (KV pages) and the step's control tensors are the
    only other device memory, all of it allocated before the first step."""

    def __init__(self, bundle_dir: str, checkpoint_dir: Optional[str], fabric: Fabric, *, max_tokens: Optional[int] = 8,
                 num_slots: int = 1, keep_logits: bool = False, parameters: Optional[Dict[str, torch.Tensor]] = None,
                 fused_head: Optional[bool] = None, fused_moe: Optional[bool] = None, l2_prefetch: Optional[bool] = None,
                 fused_gqa: Optional[bool] = None):
        """``max_tokens``: query rows per step (at most 8); ``None`` takes what the bundle's arena was planned for.
        ``parameters``: device tensors by the init plan's parameter names, used instead of a checkpoint (random-init
        benchmarks, weights another engine already holds); every parameter of the plan must be there with the plan's
        shape and dtype. ``fused_head`` / ``fused_moe``: let the dispatcher replace the instruction groups
        {q_b linear, cache write, absorb, attention} and {router, expert gate/up, expert down + all-reduce} by their
        one-launch kernels where the shapes allow, for steps of one or two rows (defaults: the head kernel for contexts up to
        2048 keys - its measured crossover; the expert block off - it measured slower than its three kernels at 1, 2 and 8 GPUs)."""
        self.fabric, self.rank, self.world = fabric, fabric.rank, fabric.world
        b = Path(bundle_dir)
        from .. import compiler

        compiler.validate_bundle(str(b))     # kernel / binding contracts of the serialized program, before any allocation
        self.program = json.loads((b / "device-program.json").read_text())
        self.manifest = json.loads((b / "serving.json").read_text())
        if self.program["parallel"]["tp"] != self.world:
            raise ValueError(f"bundle was compiled for tp={self.program['parallel']['tp']}, running on {self.world} ranks")
        init_plan = json.loads((b / f"rank-{self.rank}.init.json").read_text())
        dev = fabric.device
        self.P = (self._adopt(init_plan, parameters) if parameters is not None
                  else load_parameters(init_plan, SafetensorsDir(checkpoint_dir), dev))
        self.ins = self.program["instructions"]
        if max_tokens is None:
            planned = json.loads((b / "arena.json").read_text()).get("tokens", 1)
            max_tokens = max(1, min(8, int(planned)))
        self.T = max_tokens
        self.max_context = self.program["max_context"]
        self.page_tokens = 16
        self.max_pages = (self.max_context + self.page_tokens - 1) // self.page_tokens
        self.num_slots = num_slots
        self.num_pages = self.max_pages * num_slots
        T = self.T
        self.tokens = torch.zeros(T, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(T, dtype=torch.int32, device=dev)
        self.page_table = torch.arange(self.num_pages, dtype=torch.int32, device=dev).view(num_slots, self.max_pages).contiguous()
        self.next_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.next_vals = torch.zeros(T, dtype=torch.float32, device=dev)
        self.kps = 64
        self.max_splits = max(1, min(64, (self.max_context + self.kps - 1) // self.kps))
        while self.max_splits * self.kps < self.max_context:
            self.kps *= 2
        self.keep_logits = keep_logits
        self.logits = None
        self.vals: List[object] = [None] * len(self.ins)
        self._index_cache_of: Dict[int, torch.Tensor] = {}     # index-cache instruction -> its pages of index keys
        self._index_scales_of: Dict[int, torch.Tensor] = {}    # int8 index caches: the per-row scales
        self._index_scores = None
        self._cache_of: Dict[int, torch.Tensor] = {}     # cache-write instruction -> its pages
        self.caches: List[torch.Tensor] = []              # the same tensors in program order (one per attention layer)
        self._packed: set = set()                         # cache-write instructions whose pages hold packed int8 rows
        self._kv_of: Dict[int, tuple] = {}                # K / V append instruction -> (key pages, value pages)
        self._kv_pack = None                              # [k | v] rows of a step, for an append outside the fused group
        self._conv_state: Dict[int, torch.Tensor] = {}    # token-convolution instruction -> the previous taps-1 rows per sequence slot
        self._sink_rows: Dict[int, torch.Tensor] = {}     # sink_normalize instruction -> its rows [count, latent + rope]
        self._sinks_of: Dict[int, torch.Tensor] = {}      # cache-write instruction -> the sink rows its readers also attend to
        self.arena = FrozenArena(b, self.rank, T, dev)
        self._alloc(dev)
        self.bundle_sha256 = json.loads((b / "plan.json").read_text()).get("program_sha256", "")
        # measured at one GPU: requesting o_proj + shared expert (72 MB per layer) during the attention kernel costs 3.4 % (5.58 vs
        # 5.39 ms per step): the requests compete with the kernel's own loads. Off unless asked for; 2 = the output projection only.
        self.l2_prefetch = 0 if l2_prefetch is None else int(l2_prefetch)
        self._fused_gqa_option = fused_gqa
        # debugging aid, the device-side counterpart of the interpreter's `watch`: called as probe(instruction, rows) right after
        # each instruction was enqueued (its arena slot is still its own); not for use under graph capture
        self.probe = None
        self._prepare(fused_head, fused_moe)
        self._graph = None

    @staticmethod
    def _adopt(init_plan: dict, given: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """The caller's tensors as this rank's parameters, checked against the init plan (name, shape, dtype)."""
        out = {}
        for p in init_plan["parameters"]:
            t = given.get(p["name"])
            if t is None:
                raise KeyError(f"no tensor was given for parameter {p['name']}")
            want = {"bf16": BF16, "f32": torch.float32}.get(p["dtype"])
            if want is None or t.dtype != want or list(t.shape) != list(p["dims"]) or not t.is_contiguous():
                raise ValueError(f"parameter {p['name']}: the plan wants {p['dtype']} {p['dims']}, got {t.dtype} {list(t.shape)}")
            out[p["name"]] = t
        return out

    # -- dispatcher: instruction groups -> kernels -------------------------------------------------------
    def _prepare(self, fused_head: Optional[bool], fused_moe: Optional[bool]) -> None:
        """Finds the instruction groups that have a one-launch kernel and records them at the group's last member (the
        anchor); ``forward`` runs the anchor's kernel and skips the other members when the step is narrow enough.
        Reference: the native dispatcher that picks a kernel per instruction (native/src/token_dispatch.inc:19-294)."""
        ins = self.ins
        users: Dict[int, List[int]] = {}
        for k, i in enumerate(ins):
            for j in i["inputs"]:
                users.setdefault(j, []).append(k)

        def through_views(k: int) -> List[int]:
            out = []
            for u in users.get(k, []):
                out += through_views(u) if ins[u]["op"] == "view" else [u]
            return out

        self.head_groups: Dict[int, dict] = {}
        self.moe_groups: Dict[int, dict] = {}
        self.layer_weights: List[dict] = []       # per decoder layer, in program order: the parameter names of its kernels
        for k, i in enumerate(ins):
            if i["op"] == "mla_attention":
                kabs, kw = i["inputs"][:2]
                if len(i["inputs"]) != 2:
                    continue              # attention over a learned selection: the split-KV kernel only
                if ins[kabs]["op"] != "mla_q_absorb" or ins[kw]["op"] != "mla_kv_write":
                    continue
                kqb = ins[kabs]["inputs"][0]
                qb = ins[kqb]
                if qb["op"] != "linear" or "norm_weight" not in qb["attrs"] or "paired_weight" in qb["attrs"]:
                    continue
                vq, vlat, vr = ins[qb["inputs"][0]], ins[ins[kw]["inputs"][0]], ins[ins[kw]["inputs"][1]]
                if not all(v["op"] == "view" for v in (vq, vlat, vr)) or len({v["inputs"][0] for v in (vq, vlat, vr)}) != 1:
                    continue
                a, aa = i["attrs"], ins[kabs]["attrs"]
                q_lora, latent, rope, nope = int(vq["attrs"]["width"]), int(aa["latent"]), int(aa["rope"]), int(aa["nope"])
                vdim = int(a["value"])
                if (int(vq["attrs"]["start"]), int(vlat["attrs"]["start"]), int(vr["attrs"]["start"])) != (0, q_lora, q_lora + latent):
                    continue
                private = users.get(kqb, []) == [kabs] and users.get(kabs, []) == [k] and users.get(kw, []) == [k]
                shapes_ok = latent == 512 and rope == 64 and nope % 32 == 0 and nope <= 128 and vdim <= 128 and q_lora % 8 == 0
                self.head_groups[k] = {"members": (kqb, kw, kabs), "qkv": vq["inputs"][0], "q_lora": q_lora, "nope": nope, "vdim": vdim,
                                       "q_norm": qb["attrs"]["norm_weight"], "kv_norm": ins[kw]["attrs"]["weight"], "w_qb": qb["attrs"]["weight"],
                                       "w_kvb": a["weight"], "eps": float(qb["attrs"].get("norm_eps", 1e-5)), "theta": float(aa["theta"]),
                                       "scale": 1.0 / math.sqrt(float(a["scale_dim"])), "window": int(a["window"]), "cache": kw,
                                       "ok": private and shapes_ok and aa["weight"] == a["weight"] and ins[kw]["dtype"] == "bf16"}
            elif i["op"] == "moe_down_allreduce" and len(i["inputs"]) > 2:
                kgu, kr, kres = i["inputs"][:3]
                if ins[kgu]["op"] != "moe_gate_up" or ins[kr]["op"] != "router_topk":
                    continue
                r, g, a = ins[kr]["attrs"], ins[kgu]["attrs"], i["attrs"]
                kx = ins[kr]["inputs"][0]
                same_x = ins[kgu]["inputs"][0] == kx and kres == kx and r.get("norm_weight") == g.get("norm_weight")
                private = sorted(users.get(kr, [])) == sorted([kgu, k]) and users.get(kgu, []) == [k]
                self.moe_groups[k] = {"members": (kr, kgu), "router": kr, "gate_up": kgu, "x": kx,
                                      "ok": same_x and private and "shared_weight" in g and "shared_weight" in a}
        # grouped-query attention: {q, k, v projections of one normalised input, rotary on q and k, page append, attention} runs
        # as one packed projection + the rotate-and-append kernel + the split-KV attention (three kernels for seven instructions)
        self.gqa_groups: Dict[int, dict] = {}
        for k, i in enumerate(ins):
            if i["op"] != "paged_attention" or ins[i["inputs"][1]]["op"] != "kv_cache_append":
                continue
            kq, kc = i["inputs"]
            kk, kv = ins[kc]["inputs"]
            if ins[kq]["op"] != "rotary_prefix" or ins[kk]["op"] != "rotary_prefix" or ins[kv]["op"] != "linear":
                continue
            lq, lk = ins[kq]["inputs"][0], ins[kk]["inputs"][0]
            lins = [ins[lq], ins[lk], ins[kv]]
            if any(l["op"] != "linear" or "paired_weight" in l["attrs"] or "activation" in l["attrs"] for l in lins):
                continue
            same_src = len({l["inputs"][0] for l in lins}) == 1 and len({(l["attrs"].get("norm_weight"), l["attrs"].get("norm_eps")) for l in lins}) == 1
            rq, rk, a = ins[kq]["attrs"], ins[kk]["attrs"], i["attrs"]
            same_rope = all(rq[f] == rk[f] for f in ("head_dim", "rotary_dim", "theta")) and rq["head_dim"] == a["head_dim"]
            private = (users.get(lq, []) == [kq] and users.get(lk, []) == [kk] and users.get(kv, []) == [kc] and users.get(kq, []) == [k]
                       and users.get(kk, []) == [kc] and users.get(kc, []) == [k])
            if not (same_src and same_rope and private):
                continue
            names = [l["attrs"]["weight"] for l in lins]
            self.gqa_groups[k] = {"members": (lq, kq, lk, kk, kv, kc), "x": lins[0]["inputs"][0], "cache": kc, "weights": names,
                                  "norm": lins[0]["attrs"].get("norm_weight"), "norm_optional": "norm_optional" in lins[0]["attrs"],
                                  "eps": float(lins[0]["attrs"].get("norm_eps", 1e-5)), "rotary_dim": int(rq["rotary_dim"]), "theta": float(rq["theta"])}
        self._gqa_members = {m: k for k, g in self.gqa_groups.items() for m in g["members"]}
        self._gqa_packed: Dict[int, torch.Tensor] = {}
        for k, g in self.gqa_groups.items():
            ws = [self._param(n) for n in g["weights"]]
            adjacent = all(ws[j + 1].data_ptr() == ws[j].data_ptr() + ws[j].numel() * 2 for j in range(2)) and \
                all(w.untyped_storage().data_ptr() == ws[0].untyped_storage().data_ptr() for w in ws)
            rows = sum(w.shape[0] for w in ws)
            # the three matrices as one [q | k | v] operand: a view when the caller's tensors already sit back to back
            self._gqa_packed[k] = torch.as_strided(ws[0], (rows, ws[0].shape[1]), (ws[0].shape[1], 1)) if adjacent else torch.cat(ws, 0).contiguous()
        if self.gqa_groups:
            width = max(self._gqa_packed[k].shape[0] for k in self.gqa_groups)
            self._gqa_qkv = torch.empty(self.T, width, dtype=BF16, device=self.fabric.device)     # read by attention while the workspace holds its splits
        self.fused_gqa = bool(self.gqa_groups) and self._fused_gqa_option is not False
        self.fused_ctx_limit = 2048
        can_head = bool(self.head_groups) and all(g["ok"] for g in self.head_groups.values())
        self.fused_head = (can_head and self.max_context <= self.fused_ctx_limit) if fused_head is None else (bool(fused_head) and can_head)
        self.fuse_override: Optional[bool] = None          # engines that know the position pick the head kernel per step
        self.fused_auto = fused_head is None
        self.fused_head_rows = 2 if fused_head is None else 8      # an explicit request fuses every step width
        self.can_fuse_head = can_head
        can_moe = bool(self.moe_groups) and all(g["ok"] for g in self.moe_groups.values())
        for g in self.moe_groups.values():
            wgu = self.P.get(self.ins[g["gate_up"]]["attrs"]["weight"] + "|" + self.ins[g["gate_up"]]["attrs"]["paired_weight"])
            E = int(self.ins[g["router"]]["attrs"]["experts"])
            can_moe = can_moe and wgu is not None and wgu.shape[1] // 2 <= 1536 and E <= 256 and self.ins[g["router"]]["width"] <= 16
        self.fused_moe = False if fused_moe is None else (bool(fused_moe) and can_moe)
        self.moe_sync = None
        if can_moe:
            E = max(int(self.ins[g["router"]]["attrs"]["experts"]) for g in self.moe_groups.values())
            self.moe_sync = torch.zeros(K.moe_block_sync_words(2, E), dtype=torch.int32, device=self.fabric.device)
        self._router_shares_norm = {g["router"] for g in self.moe_groups.values() if g["ok"] and "norm_weight" in self.ins[g["router"]]["attrs"]}
        hidden = max((self.ins[self.ins[r]["inputs"][0]]["width"] for r in self._router_shares_norm), default=0)
        self.xn = self.arena.workspace(self.T * hidden * 2).view(BF16).view(self.T, hidden) if hidden else None
        # what the head kernel of a layer requests into L2 for the kernels after it: the output projection that consumes the
        # attention result and the shared expert of the layer's expert block (routed experts are not known yet)
        self._head_prefetch: Dict[int, tuple] = {}
        moe_order = sorted(self.moe_groups)
        for kh in sorted(self.head_groups):
            o = next((u for u in users.get(kh, []) if ins[u]["op"] == "linear_allreduce"), None)
            km = next((m for m in moe_order if m > kh), None)
            pf = [self.P.get(ins[o]["attrs"]["weight"])] if o is not None else []
            if km is not None and self.moe_groups[km]["ok"]:
                gu, dn = ins[self.moe_groups[km]["gate_up"]]["attrs"], ins[km]["attrs"]
                pf += [self.P.get(gu["shared_weight"] + "|" + gu["shared_paired_weight"]), self.P.get(dn["shared_weight"])]
            self._head_prefetch[kh] = tuple(t for t in pf if t is not None)
        # members of a group that the anchor's kernel covers
        self._head_members = {m: k for k, g in self.head_groups.items() for m in g["members"]}
        self._moe_members = {m: k for k, g in self.moe_groups.items() for m in g["members"]}
        per_token = self.program["launches_per_token"] + sum(1 for i in self.ins if i["op"] == "mla_attention")
        per_token += sum(1 for i in self.ins if i["op"] == "paged_attention")        # split + merge
        self.launches_per_forward = (per_token - (4 * len(self.head_groups) if self.fused_head else 0)
                                     - (2 * len(self.moe_groups) if self.fused_moe else 0) - (4 * len(self.gqa_groups) if self.fused_gqa else 0))
        self._describe()

    def _describe(self) -> None:
        """What the program says about the model, in the vocabulary of the hand-wired decoder (``models/mla_moe.py``): a
        configuration record and the parameters by role. The prompt executor (``models/mla_moe_prefill.py``) and the batch
        engine read a decoder through these attributes, so they run on a bundle's engine as they do on ``MlaMoeDecoder``.
        Left undefined (``cfg is None``) for programs that are not a stack of {latent attention, routed experts} layers."""
        self.cfg, self.w, self.kv_int8 = None, {}, bool(self._packed) and len(self._packed) == len(self._cache_of)
        ins = self.ins
        heads, moes = sorted(self.head_groups), sorted(self.moe_groups)
        emb = next((i for i in ins if i["op"] == "embedding"), None)
        head = next((i for i in ins if i["op"] == "lm_head"), None)
        if self.gqa_groups and not heads and not moes and emb is not None and head is not None:
            self._describe_dense(emb, head)
            return
        if not heads or len(heads) != len(moes) or emb is None or head is None:
            return
        from ..models.mla_moe import MlaMoeConfig

        g0, m0 = self.head_groups[heads[0]], self.moe_groups[moes[0]]
        a0, r0, gu0 = ins[heads[0]]["attrs"], ins[m0["router"]]["attrs"], ins[m0["gate_up"]]["attrs"]
        self.cfg = MlaMoeConfig(layers=len(heads), hidden=emb["width"], vocab=int(emb["attrs"]["vocab"]), heads=int(a0["heads"]),
                                q_lora=g0["q_lora"], kv_lora=int(a0["latent"]), nope=g0["nope"], rope=int(ins[g0["members"][2]]["attrs"]["rope"]),
                                vdim=g0["vdim"], experts=int(r0["experts"]), expert_ffn=ins[m0["gate_up"]]["width"], topk=int(r0["topk"]),
                                shared_ffn=int(gu0["shared_width"]) * self.world, theta=g0["theta"], eps=g0["eps"], window=g0["window"],
                                scoring=r0["scoring"], route_scale=float(r0["scale"]), eos=int(self.program.get("eos", -1)),
                                page_tokens=self.page_tokens)
        c = self.cfg
        self.hl, self.el, self.vl = c.heads // self.world, c.experts // self.world, c.vocab // self.world
        w = self.w
        w["embed"], w["final_norm"], w["lm_head"] = self._param(emb["attrs"]["weight"]), self._param(head["attrs"]["norm_weight"]), self._param(head["attrs"]["weight"])
        for l, (kh, km) in enumerate(zip(heads, moes)):
            g, m = self.head_groups[kh], self.moe_groups[km]
            qkv = ins[g["qkv"]]["attrs"]
            o = next(ins[u] for u in range(kh + 1, km) if ins[u]["op"] == "linear_allreduce" and ins[u]["inputs"][0] == kh)
            r, gu, dn = ins[m["router"]]["attrs"], ins[m["gate_up"]]["attrs"], ins[km]["attrs"]
            p = f"layers.{l}."
            w[p + "attn_norm"], w[p + "qkv_a"] = self._param(qkv["norm_weight"]), self._param(qkv["weight"] + "|" + qkv["paired_weight"])
            w[p + "q_a_norm"], w[p + "kv_a_norm"], w[p + "q_b"] = self._param(g["q_norm"]), self._param(g["kv_norm"]), self._param(g["w_qb"])
            w[p + "kv_b"] = self._param(g["w_kvb"]).view(self.hl, c.nope + c.vdim, c.kv_lora)
            w[p + "o_proj"] = self._param(o["attrs"]["weight"])
            w[p + "ffn_norm"], w[p + "router"] = self._param(r["norm_weight"]), self._param(r["weight"])
            w[p + "gate_up"], w[p + "down"] = self._param(gu["weight"] + "|" + gu["paired_weight"]), self._param(dn["weight"])
            w[p + "shared_gate_up"] = self._param(gu["shared_weight"] + "|" + gu["shared_paired_weight"])
            w[p + "shared_down"] = self._param(dn["shared_weight"])

    def _describe_dense(self, emb: dict, head: dict) -> None:
        """The same for a stack of {grouped-query attention, SwiGLU} layers, in the vocabulary of ``models/dense_gqa.py``: the
        dense prompt executor (``models/dense_prefill.py``) runs on a bundle's engine through ``cfg``, ``w``, ``hq`` / ``hk`` /
        ``vl`` and the K / V pages per layer."""
        from ..models.dense_gqa import DenseConfig

        ins, groups = self.ins, sorted(self.gqa_groups)
        a0 = ins[groups[0]]["attrs"]
        w: Dict[str, torch.Tensor] = {}
        k_cache, v_cache, ffn = [], [], 0
        for l, k in enumerate(groups):
            g, p = self.gqa_groups[k], f"layers.{l}."
            o = next((ins[u] for u in range(k + 1, len(ins)) if ins[u]["op"] == "linear_allreduce" and ins[u]["inputs"][0] == k), None)
            if o is None or g["norm"] is None:
                return
            ko = ins.index(o)
            up = next((ins[u] for u in range(ko + 1, len(ins)) if ins[u]["op"] == "linear" and ins[u]["attrs"].get("activation") == "swiglu"
                       and ins[u]["inputs"][0] == ko and "norm_weight" in ins[u]["attrs"]), None)
            down = None if up is None else next((ins[u] for u in range(ko + 1, len(ins)) if ins[u]["op"] == "linear_allreduce"
                                                 and ins[u]["inputs"][0] == ins.index(up)), None)
            if down is None:
                return
            w[p + "attn_norm"], w[p + "qkv"], w[p + "o_proj"] = self._param(g["norm"]), self._gqa_packed[k], self._param(o["attrs"]["weight"])
            w[p + "ffn_norm"] = self._param(up["attrs"]["norm_weight"])
            w[p + "gate_up"] = self._param(up["attrs"]["weight"] + "|" + up["attrs"]["paired_weight"])
            w[p + "down"] = self._param(down["attrs"]["weight"])
            ffn = int(up["attrs"]["width"]) * self.world
            kc, vc = self._kv_of[g["cache"]]
            k_cache.append(kc)
            v_cache.append(vc)
        w["embed"], w["final_norm"], w["lm_head"] = self._param(emb["attrs"]["weight"]), self._param(head["attrs"]["norm_weight"]), self._param(head["attrs"]["weight"])
        g0 = self.gqa_groups[groups[0]]
        self.cfg = DenseConfig(layers=len(groups), hidden=emb["width"], heads=int(a0["heads"]), kv_heads=int(a0["kv_heads"]), head_dim=int(a0["head_dim"]),
                               ffn=ffn, vocab=int(emb["attrs"]["vocab"]), theta=g0["theta"], eps=g0["eps"], page_tokens=self.page_tokens)
        self.w, self.k_cache, self.v_cache = w, k_cache, v_cache
        self.hq, self.hk, self.vl = self.cfg.heads // self.world, self.cfg.kv_heads // self.world, self.cfg.vocab // self.world

    def forward_feedback(self, T: Optional[int] = None) -> torch.Tensor:
        """One step whose sampled token and position + 1 become the inputs of the next step (device-side feedback)."""
        T = self.T if T is None else T
        self.forward(T)
        self.tokens[:T].copy_(self.next_ids[:T])
        self.positions[:T].add_(1)
        return self.next_ids[:T]

    # -- buffers -------------------------------------------------------------------------------------
    def _alloc(self, dev) -> None:
        """Views into the frozen arena for every instruction result; KV pages as sequence state beside it."""
        T = self.T
        max_heads, gqa_split_floats = 1, 0
        f32, i32 = torch.float32, torch.int32

        def view(k: int, shape, dtype) -> torch.Tensor:
            n = 1
            for d in shape:
                n *= d
            esize = torch.empty((), dtype=dtype).element_size()
            return self.arena.lease(k, n * esize).view(dtype).view(*shape)

        # an optional norm whose gain the checkpoint lacks passes its rows through: the compiler then gave it no slot and let
        # its source's slot live on, so the rows are handed on without a copy
        self._pass_through = {k for k, i in enumerate(self.ins) if i["op"] == "optional_norm" and k not in self.arena.slots}
        for k in self._pass_through:
            if self._param(self.ins[k]["attrs"]["weight"], True) is not None:
                raise ValueError(f"the bundle was compiled without {self.ins[k]['attrs']['weight']}, the parameters have it: recompile against this checkpoint")
        for k, i in enumerate(self.ins):
            op, w = i["op"], i["width"]
            if op == "view":
                continue
            if op == "optional_norm" and k in self._pass_through:
                continue                                                   # no slot of its own is touched
            if op == "mla_kv_write":
                if i["dtype"] == "int8_ds_mla":
                    # packed rows: 512 int8 latent values, 64 bf16 rotary values, four f32 tile scales
                    if w != 576:
                        raise NotImplementedError("the packed int8 cache holds 512 latent + 64 rotary columns")
                    self._cache_of[k] = torch.zeros(self.num_pages, self.page_tokens, 656, dtype=torch.uint8, device=dev)
                    self._packed.add(k)
                elif i["dtype"] != "bf16":
                    raise NotImplementedError(f"cache dtype {i['dtype']} has no device layout")
                else:
                    self._cache_of[k] = torch.zeros(self.num_pages, self.page_tokens, w, dtype=BF16, device=dev)
                self.caches.append(self._cache_of[k])
            elif op in ("mhc_pre", "mhc_merge"):
                S = int(i["attrs"]["streams"])
                if S + S * S > 64:
                    raise NotImplementedError("a hyper-connection slot holds at most 64 mixing weights per row")
                raw = self.arena.lease(k, T * w * 2 + T * 64 * 4)          # mixed row | post weights | stream-to-stream weights
                y = raw[:T * w * 2].view(BF16).view(T, w)
                post = raw[T * w * 2:T * w * 2 + T * S * 4].view(f32).view(T, S)
                comb = raw[T * w * 2 + T * S * 4:T * w * 2 + T * (S + S * S) * 4].view(f32).view(T, S, S)
                self.vals[k] = (y, post, comb)
            elif op == "mhc_input":
                continue                                                   # the mixed row of its hyper-connection, no copy
            elif op == "mome":
                taps = int(i["attrs"]["taps"])
                self._conv_state[k] = torch.zeros(self.num_slots, taps - 1, w, dtype=BF16, device=dev)
                self.vals[k] = view(k, (T, w), BF16)
            elif op == "sink_normalize":
                # the sink rows depend on parameters only: normalised once, kept beside the cache they belong to
                a = i["attrs"]
                count, lat, rope = int(a["count"]), int(a["latent"]), int(a["rope"])
                rows = torch.empty(count, lat + rope, dtype=BF16, device=dev)
                K.rmsnorm(self._param(a["weight"] + ".param_sink_compressed_kv"), self._param(a["norm"]), float(a["eps"]), out=rows[:, :lat])
                rows[:, lat:].copy_(self._param(a["weight"] + ".param_sink_k_pe"))
                self._sink_rows[k] = rows
            elif op == "kv_cache_append":
                if i["attrs"].get("cache_dtype", "bf16") != "bf16":
                    raise NotImplementedError("a compiled program's K / V pages are bf16")
                hd = int(i["attrs"]["head_dim"])
                kvl = w // (2 * hd)
                pages = [torch.zeros(self.num_pages, self.page_tokens, kvl, hd, dtype=BF16, device=dev) for _ in range(2)]
                self._kv_of[k] = tuple(pages)
                if self._kv_pack is None or self._kv_pack.shape[1] < w:
                    self._kv_pack = torch.empty(T, w, dtype=BF16, device=dev)
            elif op == "paged_attention":
                gqa_split_floats = max(gqa_split_floats, (int(i["attrs"]["heads"]) // self.world) * (int(i["attrs"]["head_dim"]) + 2))
                if int(i["attrs"].get("window", 0)) not in (0,) and int(i["attrs"]["window"]) < self.max_context:
                    raise NotImplementedError("windowed grouped-query attention has no device kernel")
                self.vals[k] = view(k, (T, w), BF16)
            elif op == "index_cache_append":
                kind = i["attrs"].get("cache_dtype", "bf16")
                if kind == "int8":
                    # int8 keys with one half-precision scale per row (the selector quantises the query heads the same way)
                    self._index_cache_of[k] = torch.zeros(self.num_pages, self.page_tokens, w, dtype=torch.int8, device=dev)
                    self._index_scales_of[k] = torch.zeros(self.num_pages, self.page_tokens, dtype=torch.float16, device=dev)
                elif kind == "bf16":
                    self._index_cache_of[k] = torch.zeros(self.num_pages, self.page_tokens, w, dtype=BF16, device=dev)
                else:
                    raise NotImplementedError(f"index cache dtype {kind} has no device layout")
            elif op == "sparse_index":
                self.vals[k] = view(k, (T, w), i32)
                self._index_scores = torch.empty(T, self.max_context, dtype=f32, device=dev)      # selector scratch: one score per key
            elif op == "router_topk":
                E = int(i["attrs"]["experts"])
                raw = self.arena.lease(k, T * w * 8 + T * E * 4)           # ids | weights | logits, one slot
                ids = raw[:T * w * 4].view(i32).view(T, w)
                wts = raw[T * w * 4:T * w * 8].view(f32).view(T, w)
                logits = raw[T * w * 8:].view(f32).view(T, E)
                self.vals[k] = (ids, wts, logits)
            elif op == "moe_gate_up":
                topk = self.ins[i["inputs"][1]]["width"]
                self.vals[k] = view(k, (T, topk + 1, w), BF16)
                self.vals[k].zero_()
            elif op == "mla_q_absorb":
                a = i["attrs"]
                hl = int(a["heads"]) // self.world
                max_heads = max(max_heads, hl)
                self.vals[k] = view(k, (T, hl, int(a["latent"]) + int(a["rope"])), BF16)
            elif op == "lm_head":
                vl = int(i["attrs"]["width"])
                self._partial_floats = ((vl + 7) // 8) * 8 * 2
                if self.keep_logits:
                    self.logits = torch.empty(T, vl, dtype=torch.float32, device=dev)
                self.vals[k] = self.next_ids
            else:
                self.vals[k] = view(k, (T, w), f32 if i["dtype"] == "f32" else BF16)
        head = next((i for i in self.ins if i["op"] == "lm_head"), None)
        self.x = self.vals[head["inputs"][0]] if head is not None else None      # the final hidden rows (before the last norm)
        # kernel scratch comes out of the frozen workspace: the attention splits and the argmax partials never live at once
        has_latent = any(i["op"] == "mla_attention" for i in self.ins)
        self.scratch = self.arena.workspace(T * self.max_splits * max(max_heads * (512 + 2) if has_latent else 0, gqa_split_floats, 1) * 4).view(f32)
        self.partial = self.arena.workspace(self._partial_floats * 4).view(f32)

    def _param(self, name: str, optional: bool = False):
        if name in self.P:
            return self.P[name]
        if optional:
            return None
        raise KeyError(f"bundle has no parameter {name}")

    # -- one step --------------------------------------------------------------------------------------
    def forward(self, T: Optional[int] = None) -> torch.Tensor:
        T = self.T if T is None else T
        fab, st = self.fabric, self.fabric.desc.status
        tok, pos, slot = self.tokens[:T], self.positions[:T], self.slots[:T]
        V = self.vals

        def val(idx):
            v = V[idx]
            return v[:T] if isinstance(v, torch.Tensor) else v

        head = (self.fused_head if self.fuse_override is None else (self.fuse_override and self.can_fuse_head)) and T <= self.fused_head_rows
        moe = self.fused_moe and T <= 2
        gqa = self.fused_gqa
        probe = self.probe
        for k, i in enumerate(self.ins):
            op, a, ins = i["op"], i["attrs"], i["inputs"]
            if probe is not None and k:
                probe(k - 1, T)
            if (head and k in self._head_members) or (moe and k in self._moe_members) or (gqa and k in self._gqa_members):
                if op in ("mla_kv_write", "kv_cache_append"):
                    V[k] = k                  # the cache of this write, for whoever reads it
                continue
            norm_w = self._param(a["norm_weight"], "norm_optional" in a) if "norm_weight" in a else None
            eps = float(a.get("norm_eps", 1e-5))
            if head and k in self.head_groups:
                g = self.head_groups[k]
                hl = int(a["heads"]) // self.world
                K.mla_head_decode(val(g["qkv"]), self._param(g["q_norm"]), self._param(g["kv_norm"]), self._param(g["w_qb"]),
                                  self._param(g["w_kvb"]).view(hl, g["nope"] + g["vdim"], 512), self._cache_of[g["cache"]], pos, slot,
                                  self.page_table, q_lora=g["q_lora"], nope=g["nope"], scale=g["scale"], eps=g["eps"], theta=g["theta"],
                                  window=g["window"], out=val(k), status_ptr=st, prefetch=self._head_prefetch.get(k, ())[:1 if self.l2_prefetch == 2 else 3] if self.l2_prefetch else ())
            elif moe and k in self.moe_groups:
                g = self.moe_groups[k]
                r, gu = self.ins[g["router"]]["attrs"], self.ins[g["gate_up"]]["attrs"]
                ids, wts, logits = V[g["router"]]
                wgu, wd = self._param(gu["weight"] + "|" + gu["paired_weight"]), self._param(a["weight"])
                K.moe_block(val(g["x"]), self._param(r["weight"]), wgu, wd, self.rank * wgu.shape[0], int(r["topk"]), fab, sync=self.moe_sync,
                            norm_w=self._param(r["norm_weight"]) if "norm_weight" in r else None, eps=float(r.get("norm_eps", 1e-5)),
                            bias=self._param(r["weight"] + ".e_score_correction_bias", True), scoring=r["scoring"],
                            renorm=r.get("renorm", "true") != "false", scale=float(r["scale"]),
                            w_shared_gu=self._param(gu["shared_weight"] + "|" + gu["shared_paired_weight"]),
                            w_shared_down=self._param(a["shared_weight"]), logits=logits[:T], ids=ids[:T], wts=wts[:T],
                            act=V[g["gate_up"]][:T], out=val(k))
            elif gqa and k in self.gqa_groups:
                g = self.gqa_groups[k]
                H, KVH, hd = int(a["heads"]) // self.world, int(a["kv_heads"]) // self.world, int(a["head_dim"])
                wq = self._gqa_packed[k]
                qkv = self._gqa_qkv[:T, :wq.shape[0]]
                kc, vc = self._kv_of[g["cache"]]
                K.gemv(val(g["x"]), wq, norm_w=self._param(g["norm"], g["norm_optional"]) if g["norm"] else None, eps=g["eps"], out=qkv)
                K.gqa_rope_kv_write(qkv, pos, slot, self.page_table, kc, vc, heads=H, kv_heads=KVH, head_dim=hd, rotary_dim=g["rotary_dim"],
                                    theta=g["theta"], status_ptr=st)
                K.gqa_decode_attention(qkv, kc, vc, pos, slot, self.page_table, heads=H, kv_heads=KVH, head_dim=hd, scale=float(a["scale"]),
                                       keys_per_split=self.kps, max_splits=self.max_splits, scratch=self.scratch, out=val(k), status_ptr=st)
            elif op == "kv_cache_append":
                # k and v rows side by side in the pack buffer, then the append kernel with no query heads and no rotation
                kr, vr = val(ins[0]), val(ins[1])
                kc, vc = self._kv_of[k]
                pack = self._kv_pack[:T, :kr.shape[1] + vr.shape[1]]
                pack[:, :kr.shape[1]].copy_(kr)
                pack[:, kr.shape[1]:].copy_(vr)
                K.gqa_rope_kv_write(pack, pos, slot, self.page_table, kc, vc, heads=0, kv_heads=kc.shape[2], head_dim=kc.shape[3], rotary_dim=0,
                                    theta=2.0, status_ptr=st)
                V[k] = k
            elif op == "paged_attention":
                kc, vc = self._kv_of[V[ins[1]]]
                K.gqa_decode_attention(val(ins[0]), kc, vc, pos, slot, self.page_table, heads=int(a["heads"]) // self.world,
                                       kv_heads=kc.shape[2], head_dim=kc.shape[3], scale=float(a["scale"]), keys_per_split=self.kps,
                                       max_splits=self.max_splits, scratch=self.scratch, out=val(k), status_ptr=st)
            elif op == "embedding":
                K.embedding(tok, self._param(a["weight"]), out=val(k), status_ptr=st)
            elif op == "view":
                src = V[ins[0]]
                s, w = int(a["start"]), int(a["width"])
                V[k] = src[:, s:s + w]
            elif op == "linear":
                name = a["weight"] + ("|" + a["paired_weight"] if "paired_weight" in a else "")
                K.gemv(val(ins[0]), self._param(name), norm_w=norm_w, eps=eps, swiglu=a.get("activation") == "swiglu", out=val(k))
            elif op == "linear_allreduce":
                res = val(ins[1]) if len(ins) > 1 else None
                K.gemv_allreduce(val(ins[0]), self._param(a["weight"]), fab, residual=res, out=val(k))
            elif op == "norm":
                K.rmsnorm(val(ins[0]), self._param(a["weight"]), float(a["eps"]), out=val(k))
            elif op == "mla_kv_write":
                lat, kr = val(ins[0]), val(ins[1])
                if len(ins) > 2:
                    self._sinks_of[k] = self._sink_rows[ins[2]]
                V[k] = k
                if kr.data_ptr() != lat.data_ptr() + lat.shape[1] * 2 or kr.stride(0) != lat.stride(0):
                    # e.g. a convolved latent and the raw rope columns of the projection: the kernel reads them where they are
                    write = K.mla_kv_write_q8_split if k in self._packed else K.mla_kv_write_split
                    write(lat, kr, self._param(a["weight"]), pos, slot, self.page_table, self._cache_of[k], eps=float(a["eps"]),
                          theta=float(a["theta"]), status_ptr=st)
                    continue
                kv = torch.as_strided(lat, (T, lat.shape[1] + kr.shape[1]), (lat.stride(0), 1))
                if k in self._packed:
                    K.mla_kv_write_q8(kv, self._param(a["weight"]), pos, slot, self.page_table, self._cache_of[k], eps=float(a["eps"]),
                                      theta=float(a["theta"]), status_ptr=st)
                    continue
                K.mla_kv_write(kv, self._param(a["weight"]), pos, slot, self.page_table, self._cache_of[k], latent=lat.shape[1],
                               rope=kr.shape[1], eps=float(a["eps"]), theta=float(a["theta"]), status_ptr=st)
                V[k] = k
            elif op == "mla_q_absorb":
                H, nope, rope, latent = int(a["heads"]), int(a["nope"]), int(a["rope"]), int(a["latent"])
                vdim = int(a.get("value", nope))
                w = self._param(a["weight"]).view(H // self.world, nope + vdim, latent)
                K.mla_q_absorb(val(ins[0]), w, pos, nope=nope, rope=rope, theta=float(a["theta"]), out=val(k))
            elif op == "rotary_prefix":
                HC.rope_prefix(val(ins[0]), pos, heads=int(a["heads"]), head_dim=int(a["head_dim"]), rotary_dim=int(a["rotary_dim"]),
                               theta=float(a["theta"]), out=val(k))
            elif op == "index_cache_append":
                HC.index_cache_append(val(ins[0]), self._index_cache_of[k], pos, slot, self.page_table, status_ptr=st,
                                      scales=self._index_scales_of.get(k))
                V[k] = k
            elif op == "sparse_index":
                Hi, dim = int(a["heads"]), int(a["head_dim"])
                q = val(ins[0])
                if not q.is_contiguous():
                    raise NotImplementedError("the index query must be a whole instruction result")
                HC.sparse_index(q.view(T, Hi, dim), val(ins[1]), self._index_cache_of[V[ins[2]]], pos, slot, self.page_table,
                                ctx=self.max_context, topk=int(a["topk"]), status_ptr=st, scores=self._index_scores[:T], out=val(k),
                                key_scales=self._index_scales_of.get(V[ins[2]]))
            elif op == "add":
                HC.add_rows(val(ins[0]), val(ins[1]), out=val(k))
            elif op == "swiglu":
                if len(ins) == 2:
                    HC.swiglu_pair(val(ins[0]), val(ins[1]), out=val(k))
                else:
                    gu = val(ins[0])
                    HC.swiglu_pair(gu[:, :gu.shape[1] // 2], gu[:, gu.shape[1] // 2:], out=val(k))
            elif op == "repeat":
                n = int(a["count"])
                x = val(ins[0])
                val(k).view(T, n, x.shape[1]).copy_(x.unsqueeze(1).expand(T, n, x.shape[1]))
            elif op == "cast":
                val(k).copy_(val(ins[0]))
            elif op == "optional_norm":
                w = self._param(a["weight"], True)
                if w is None and k in self._pass_through:
                    V[k] = V[ins[0]]               # the checkpoint has no such gain and the source's slot stays intact for as long
                                                   # as this value is read: the rows pass through without a copy
                elif w is None:
                    val(k).copy_(val(ins[0]))      # ... otherwise into this instruction's own slot
                else:
                    K.rmsnorm(val(ins[0]), w, float(a["eps"]), out=val(k))
            elif op in ("mhc_pre", "mhc_merge"):
                S = int(a["streams"])
                y, post, comb = V[k]
                X = val(ins[0])
                b = a["weight"]
                HC.mhc_pre(X.view(T, S, X.shape[1] // S), self._param(b + ".phi"), self._param(b + ".gamma"), self._param(b + ".alpha"),
                           self._param(b + ".beta"), sinkhorn=int(a["sinkhorn"]), eps=float(a["eps"]), out=(y[:T], post[:T], comb[:T]),
                           tickets_ptr=fab.ticket_ptr + 32 if T <= 8 else None)        # eight ticket words after the router's
            elif op == "mhc_input":
                V[k] = V[ins[0]][0]
            elif op == "mhc_post":
                _, post, comb = V[ins[0]]
                S = post.shape[1]
                X, Y = val(ins[2]), val(k)
                HC.mhc_post(X.view(T, S, X.shape[1] // S), val(ins[1]), post[:T], comb[:T], out=Y.view(T, S, Y.shape[1] // S), norm_w=norm_w, eps=eps)
            elif op == "mome":
                w = self._param(a["weight"])
                x = val(ins[0])
                HC.mome(x, w, self._conv_state[k], pos, slot, c_offset=self.rank * x.shape[1] if a.get("placement") == "tp_channels" else 0,
                        out=val(k))
            elif op == "sink_normalize":
                V[k] = self._sink_rows[k]
            elif op == "mla_attention":
                H, latent, vdim = int(a["heads"]), int(a["latent"]), int(a["value"])
                nope = int(a.get("nope", vdim))
                w = self._param(a["weight"]).view(H // self.world, nope + vdim, latent)
                cache = self._cache_of[V[ins[1]]]
                K.mla_decode_attention(val(ins[0]), cache, pos, slot, self.page_table, w, nope=nope,
                                       scale=1.0 / math.sqrt(float(a["scale_dim"])), window=int(a["window"]),
                                       keys_per_split=self.kps, max_splits=self.max_splits, scratch=self.scratch,
                                       out=val(k), status_ptr=st, indices=val(ins[2]) if len(ins) > 2 else None,
                                       sinks=self._sinks_of.get(V[ins[1]]), packed=V[ins[1]] in self._packed)
            elif op == "router_topk":
                ids, wts, logits = V[k]
                # when the expert kernels read the same rows under the same norm, the router leaves the normalised rows in the
                # workspace and they skip their own RMSNorm prologue
                shares = k in self._router_shares_norm
                K.router_topk(val(ins[0]), self._param(a["weight"]), int(a["topk"]), norm_w=norm_w, eps=eps,
                              scoring=a["scoring"], scale=float(a["scale"]), renorm=a.get("renorm", "true") != "false",
                              bias=self._param(a["weight"] + ".e_score_correction_bias", True), ticket_ptr=fab.ticket_ptr,
                              logits=logits[:T], ids=ids[:T], wts=wts[:T], xn=self.xn[:T] if shares else None)
            elif op == "moe_gate_up":
                ids = V[ins[1]][0][:T]
                wgu = self._param(a["weight"] + "|" + a["paired_weight"])
                sh = self._param(a["shared_weight"] + "|" + a["shared_paired_weight"]) if "shared_weight" in a else None
                if ins[1] in self._router_shares_norm:
                    K.moe_gate_up(self.xn[:T], ids, wgu, self.rank * wgu.shape[0], w_shared_gu=sh, act=V[k][:T])
                else:
                    K.moe_gate_up(val(ins[0]), ids, wgu, self.rank * wgu.shape[0], norm_w=norm_w, eps=eps, w_shared_gu=sh, act=V[k][:T])
            elif op == "moe_down_allreduce":
                ids, wts, _ = V[ins[1]]
                wd = self._param(a["weight"])
                sh = self._param(a["shared_weight"]) if "shared_weight" in a else None
                res = val(ins[2]) if len(ins) > 2 else None
                K.moe_down_allreduce(V[ins[0]][:T], ids[:T], wts[:T], wd, self.rank * wd.shape[0], fab, w_shared_down=sh,
                                     residual=res, out=val(k))
            elif op == "lm_head":
                w = self._param(a["weight"])
                K.lm_head_argmax(val(ins[0]), w, fab, norm_w=norm_w, eps=eps, vocab_offset=self.rank * w.shape[0],
                                 partial=self.partial, logits=None if self.logits is None else self.logits[:T],
                                 out_ids=self.next_ids[:T], out_vals=self.next_vals[:T])
            else:
                raise NotImplementedError(f"no device kernel bound for instruction '{op}' ({i['name']})")
        if probe is not None:
            probe(len(self.ins) - 1, T)
        return self.next_ids[:T]

    def capture(self, T: Optional[int] = None, feedback: bool = False) -> torch.cuda.CUDAGraph:
        """One step as a CUDA graph (after an eager warm-up run of the same step); with ``feedback`` the graph also feeds the
        sampled token and position + 1 back into the input buffers."""
        T = self.T if T is None else T
        self.forward(T)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            if feedback:
                self.forward_feedback(T)
            else:
                self.forward(T)
        self._graph = g
        return g

    def reset(self) -> None:
        for c in list(self.caches) + list(self._index_cache_of.values()) + list(self._index_scales_of.values()) + [t for kv in self._kv_of.values() for t in kv] + list(self._conv_state.values()):
            c.zero_()
