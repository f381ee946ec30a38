"""torchrun worker for the pipeline-parallel tests: XFT_PIPELINE_STAGE stages, rank 0 drives, the others follow."""
import sys

import torch
import torch.distributed as dist

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
g = torch.Generator().manual_seed(1)
ids = torch.randint(0, 32000, (int(sys.argv[3]) if len(sys.argv) > 3 else 2, 32), generator=g)
m = model.model
if model.rank == 0:
    sid = model.set_input_cb(ids.tolist(), None, 64)
    logits = model.forward_cb()
    model.free_seqs(sid)
    tokens = model.generate(ids, max_length=48)
else:
    model.set_input_cb()
    model.forward_cb()
    model.free_seqs()
    model.generate()
layers = [None] * dist.get_world_size()
dist.all_gather_object(layers, (m.decoder.l0, m.decoder.l1, m.ctx.pp_rank, m.ctx.tp_rank))
if model.rank == 0:
    torch.save({"logits": logits.float().cpu(), "tokens": tokens.cpu(), "layers": layers,
                "microbatches": getattr(m, "pp_microbatches", 0)}, out)
m._closed = True
dist.barrier()
