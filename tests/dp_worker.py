"""torchrun worker for the data-parallel attention test (XFT_ATTENTION_DP=1): rank 0 drives, the others follow.
Scenarios: one sequence (the other rank has no tokens and only serves its experts), three prompts of different length
with a small XFT_MAX_BATCH_TOKENS (the ranks need different numbers of prefill passes), beam search, all-position
logits."""
import sys

import torch
import torch.distributed as dist

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
m = model.model
g = torch.Generator().manual_seed(4)
one = torch.randint(0, 1000, (1, 9), generator=g)
three = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 7, 33)]
two = torch.randint(0, 1000, (2, 11), generator=g)
res = {}
if model.rank == 0:
    res["one"] = model.generate(one, max_length=15)
    sid = model.set_input_cb(three, None, 64)
    res["three"] = model.forward_cb()
    model.free_seqs(sid)
    res["beams"] = model.generate(two, max_length=16, num_beams=2)
    res["all"] = model(two)
else:
    model.generate()
    model.set_input_cb()
    model.forward_cb()
    model.free_seqs()
    model.generate()
    model(None)
info = [None] * dist.get_world_size()
dist.all_gather_object(info, (m.ctx.dp_size, m.ctx.tp_size, m.ctx.stats["all_to_all"], m.decoder.layers[0].o.in_features))
if model.rank == 0:
    res["info"] = info
    torch.save(res, out)
m._closed = True
dist.barrier()
