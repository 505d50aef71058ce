"""Engine worker: the GPU side of ``ifab-server``.

One worker process per GPU (plain ``python -m ...`` for one GPU, under ``torch.distributed.run`` for tensor /
expert parallel models). Rank 0 connects to the Unix socket in ``IFAB_ENGINE_SOCKET`` and answers the server's
newline-delimited JSON requests (``info`` / ``admit`` / ``step`` / ``release`` / ``shutdown``); every request is
broadcast to the other ranks so that all of them launch the same kernels (the collectives live inside those
kernels). A ``step`` carries slices ``[resident, position, count, sample]`` of several sequences: prompt chunks and
decode rows are packed into launches of up to ``max_tokens`` rows (continuous batching); one token per sampling
slice goes back. Sequence slot ``resident`` owns the pages ``resident * max_pages ...`` of the KV cache.

    IFAB_ENGINE_SOCKET=/tmp/e.sock python -m ironpangu_b200.runtime.engine_worker --model tiny --max-num-seqs 4

Reference: the ResidentEngine trait and its packed batch path (frontend/src/program_worker.rs:22-61,279-317).
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import sys
from typing import Dict, List

import torch
import torch.distributed as dist


class BatchEngine:
    """Packs the slices of one scheduler step into decoder launches; greedy sampling on the device."""

    def __init__(self, decoder, model_name: str, context: int, vocab: int, eos: int = -1, greedy_only: bool = True):
        self.dec, self.name, self.context, self.eos, self.vocab = decoder, model_name, context, eos, vocab
        self.greedy_only = greedy_only
        self.residents = decoder.num_slots
        self.rows = decoder.T
        self._host = torch.zeros(3, self.rows, dtype=torch.int32).pin_memory()
        self._out = torch.zeros(self.rows, dtype=torch.int32).pin_memory()
        self.next_pos = [0] * self.residents

    def info(self) -> Dict:
        return {"model": self.name, "residents": self.residents, "token_budget": self.rows, "chunk": self.rows,
                "context": self.context, "vocab": self.vocab, "eos": max(self.eos, 0), "has_eos": self.eos >= 0,
                "world": self.dec.world, "greedy_only": self.greedy_only}

    def admit(self, resident: int, sampling: Dict, reserve: int) -> None:
        if not 0 <= resident < self.residents:
            raise ValueError("resident out of range")
        if reserve > self.context:
            raise OverflowError("request does not fit the sequence slot")
        if self.greedy_only and float(sampling.get("temperature", 0.0)) > 0.0 and int(sampling.get("top_k", 0)) != 1:
            raise ValueError("this engine samples greedily only")
        self.next_pos[resident] = 0

    def release(self, resident: int) -> None:
        self.next_pos[resident] = 0

    def step(self, slices: List[List[int]], tokens: List[int]) -> List[int]:
        d = self.dec
        rows = []                     # (token, position, slot, slice index or -1 when the row does not sample)
        off = 0
        for i, (resident, position, count, sample) in enumerate(slices):
            if position != self.next_pos[resident]:
                raise RuntimeError(f"slice of resident {resident} starts at {position}, expected {self.next_pos[resident]}")
            if position + count > self.context:
                raise RuntimeError("slice runs past the context")
            for k in range(count):
                last = k == count - 1
                rows.append((tokens[off + k], position + k, resident, i if (sample and last) else -1))
            off += count
            self.next_pos[resident] = position + count
        out = [0] * len(slices)
        for r0 in range(0, len(rows), self.rows):
            part = rows[r0:r0 + self.rows]
            n = len(part)
            for j, (tok, pos, slot, _) in enumerate(part):
                self._host[0, j], self._host[1, j], self._host[2, j] = tok, pos, slot
            d.tokens[:n].copy_(self._host[0, :n], non_blocking=True)
            d.positions[:n].copy_(self._host[1, :n], non_blocking=True)
            d.slots[:n].copy_(self._host[2, :n], non_blocking=True)
            d.forward(n)
            self._out[:n].copy_(d.next_ids[:n], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            for j, (_, _, _, si) in enumerate(part):
                if si >= 0:
                    out[si] = int(self._out[j])
        if d.fabric.status() != 0:
            raise RuntimeError(f"kernel status word = {d.fabric.status()}")
        return out


def build_engine(args, rank: int, world: int) -> BatchEngine:
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.parallel.fabric import Fabric

    dev = torch.device("cuda", torch.cuda.current_device())
    fab = Fabric(rank, world)
    if args.bundle:
        # a compiled bundle + its checkpoint: the physical program is executed instruction by instruction
        from ironpangu_b200.runtime.plan_engine import PlanEngine

        eng = PlanEngine(args.bundle, args.checkpoint, fab, max_tokens=8, num_slots=args.max_num_seqs)
        head = [i for i in eng.ins if i["op"] == "lm_head"][-1]
        vocab = int(eng._param(head["attrs"]["weight"]).shape[0]) * world
        return BatchEngine(eng, os.path.basename(os.path.normpath(args.bundle)), min(args.max_model_len, eng.max_context), vocab)
    cfg = MlaMoeConfig.tiny(args.layers or 2) if args.model == "tiny" else MlaMoeConfig.flagship()
    if args.model != "tiny" and args.layers:
        cfg.layers = args.layers
    weights = random_rank_weights(cfg, rank, world, dev, seed=args.seed)
    dec = MlaMoeDecoder(cfg, weights, fab, max_tokens=8, max_context=args.max_model_len, num_slots=args.max_num_seqs)
    return BatchEngine(dec, f"ifab-{args.model}", args.max_model_len, cfg.vocab, eos=cfg.eos)


def serve(engine: BatchEngine, rank: int, world: int, sock_path: str) -> None:
    conn = None
    buf = b""
    if rank == 0:
        conn = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        conn.connect(sock_path)
    while True:
        req = None
        if rank == 0:
            while b"\n" not in buf:
                chunk = conn.recv(1 << 16)
                if not chunk:
                    req = {"op": "shutdown"}
                    break
                buf += chunk
            if req is None:
                line, buf = buf.split(b"\n", 1)
                req = json.loads(line)
        if world > 1:
            box = [req]
            dist.broadcast_object_list(box, src=0)
            req = box[0]
        op = req.get("op")
        try:
            if op == "info":
                resp = {"ok": True, "info": engine.info()}
            elif op == "admit":
                engine.admit(int(req["resident"]), req.get("sampling", {}), int(req.get("reserve", 0)))
                resp = {"ok": True}
            elif op == "step":
                resp = {"ok": True, "tokens": engine.step(req["slices"], req["tokens"])}
            elif op == "release":
                engine.release(int(req["resident"]))
                resp = {"ok": True}
            elif op == "shutdown":
                resp = {"ok": True}
            else:
                resp = {"ok": False, "kind": "invalid", "error": f"unknown op {op!r}"}
        except OverflowError as e:
            resp = {"ok": False, "kind": "capacity", "error": str(e)}
        except ValueError as e:
            resp = {"ok": False, "kind": "invalid", "error": str(e)}
        except Exception as e:  # noqa: BLE001 - every failure must reach the server as a backend error
            resp = {"ok": False, "kind": "backend", "error": f"{type(e).__name__}: {e}"}
        if rank == 0 and conn is not None:
            try:
                conn.sendall(json.dumps(resp).encode() + b"\n")
            except OSError:
                op = "shutdown"
        if op == "shutdown":
            break
    if conn is not None:
        conn.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny", choices=["tiny", "flagship"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--bundle", default="")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--max-num-seqs", type=int, default=4)
    ap.add_argument("--max-model-len", type=int, default=256)
    ap.add_argument("--socket", default=os.environ.get("IFAB_ENGINE_SOCKET", ""))
    args = ap.parse_args()
    if not args.socket:
        raise SystemExit("no engine socket: set IFAB_ENGINE_SOCKET or pass --socket")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    engine = build_engine(args, rank, world)
    try:
        serve(engine, rank, world, args.socket)
    finally:
        torch.cuda.synchronize()
        engine.dec.fabric.close()
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
