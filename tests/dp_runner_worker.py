"""torchrun worker: the data-parallel decode runner (CudaRunner._step_dp) on CPU ranks.  The CUDA-graph parts are
replaced by eager stand-ins (_step_local runs the decoder on the local sequences, _step_idle serves the experts), so
what is checked is the division of the batch, the idle rank and the token exchange."""
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist

import xfastertransformer_b200 as xft
from xfastertransformer_b200.runtime import sampler as S
from xfastertransformer_b200.runtime.cuda_runner import CudaRunner

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
m = model.model


class EagerRunner:
    enabled = True
    bucket = staticmethod(CudaRunner.bucket)
    can_run = CudaRunner.can_run
    step = CudaRunner.step
    _step_dp = CudaRunner._step_dp

    def __init__(self, eng):
        self.m = eng
        self.steps = self.idle_steps = 0

    def reset(self):
        pass

    def _step_local(self, seqs, cfg):
        self.steps += 1
        with torch.no_grad():
            local = self.m.decoder.forward(self.m.make_batch(seqs), self.m.cache)
        return S.greedy_select(local, self.m.decoder.v0, self.m.ctx).cpu().tolist()

    def _step_idle(self):
        self.idle_steps += 1
        with torch.no_grad():
            self.m.decoder.forward_idle()
        return []


m.ctx.epcomm = SimpleNamespace(max_tokens=64, fits=lambda T, k: False)       # lets can_run through; the exchange stays on gloo
m.runner = EagerRunner(m)
g = torch.Generator().manual_seed(4)
one = torch.randint(0, 1000, (1, 9), generator=g)
three = torch.randint(0, 1000, (3, 11), generator=g)
res = {}
if model.rank == 0:
    res["one"] = model.generate(one, max_length=15)
    res["three"] = model.generate(three, max_length=17)
else:
    model.generate()
    model.generate()
stats = [None] * dist.get_world_size()
dist.all_gather_object(stats, (m.runner.steps, m.runner.idle_steps))
if model.rank == 0:
    res["stats"] = stats
    torch.save(res, out)
m._closed = True
dist.barrier()
