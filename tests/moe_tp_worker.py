"""torchrun worker for the MoE multi-rank test: rank 0 drives, the others follow; saves rank 0's last-position logits
and how many experts each rank holds."""
import sys

import torch
import torch.distributed as dist

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
ids = torch.randint(0, 1000, (3, 20), generator=torch.Generator().manual_seed(2))
m = model.model
if model.rank == 0:
    sid = model.set_input_cb(ids.tolist(), None, 64)
    logits = model.forward_cb()
    nxt = logits.argmax(-1).tolist()
    model.set_input_cb(nxt, sid, 64)           # one decode step on top of the prefill
    logits2 = model.forward_cb()
    model.free_seqs(sid)
else:
    model.set_input_cb()
    model.forward_cb()
    model.set_input_cb()
    model.forward_cb()
    model.free_seqs()
moe_layer = next(L for L in m.decoder.layers if getattr(L, "experts", None))
held = [None] * dist.get_world_size()
dist.all_gather_object(held, (len(moe_layer.experts), moe_layer.e0, moe_layer.experts[0][1].in_features))
if model.rank == 0:
    torch.save({"logits": logits, "logits2": logits2, "held": held}, out)
m._closed = True
dist.barrier()
