"""Two CPU ranks (gloo) run the engine worker's request loop over a fake engine; rank 0 talks to the test through a Unix
socket. Scenario from argv: agree | mismatch | raise, then the agreement mode (strict | deferred). Run under torch.distributed.run."""
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class FakeEngine:
    def __init__(self, rank, scenario):
        self.rank, self.scenario, self.steps = rank, scenario, 0

    def info(self):
        return {"model": "fake", "residents": 2, "token_budget": 8, "chunk": 8, "context": 64, "vocab": 100, "eos": 0, "has_eos": False,
                "world": 2, "greedy_only": True}

    def admit(self, resident, sampling, reserve):
        if reserve > 64:
            raise OverflowError("request does not fit the sequence slot")

    def release(self, resident):
        pass

    def audit(self):
        return {"steps": self.steps}

    def step(self, slices, tokens):
        self.steps += 1
        if self.scenario == "raise" and self.rank == 1 and self.steps == 2:
            raise RuntimeError("rank-local failure")
        out = [(sum(tokens) + i) % 100 for i in range(len(slices))]
        if self.scenario == "mismatch" and self.rank == 1 and self.steps == 2:
            out[0] = (out[0] + 1) % 100
        return out


def main():
    from ironpangu_b200.runtime.engine_worker import serve

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    mode = sys.argv[2] if len(sys.argv) > 2 else "strict"
    serve(FakeEngine(rank, sys.argv[1]), rank, world, os.environ["IFAB_ENGINE_SOCKET"], None, mode)
    dist.destroy_process_group()
    print(f"rank {rank} left the loop", flush=True)


if __name__ == "__main__":
    main()
