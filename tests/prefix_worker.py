"""torchrun worker: automatic prefix reuse (XFT_PREFIX_CACHE=1) under tensor parallelism; rank 0 drives two prompts that
share a long prefix, the other rank follows; every rank must adopt the same cached blocks."""
import sys

import torch
import torch.distributed as dist

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
g = torch.Generator().manual_seed(11)
common = torch.randint(5, 900, (150,), generator=g).tolist()
p1 = common + [3, 4, 5]
p2 = common + torch.randint(5, 900, (20,), generator=g).tolist()
if model.rank == 0:
    sid = model.set_input_cb([p1], None, 256)
    model.forward_cb()
    model.free_seqs(sid)
    sid = model.set_input_cb([p2], None, 256)
    logits = model.forward_cb()
    model.free_seqs(sid)
    tokens = model.generate(torch.tensor([p2]), max_length=len(p2) + 5)
else:
    for _ in range(2):
        model.set_input_cb()
        model.forward_cb()
        model.free_seqs()
    model.generate()
idx = model.model.cache.prefix_index
stats = [None] * dist.get_world_size()
dist.all_gather_object(stats, (idx.hit_blocks, len(idx.entries)))
if model.rank == 0:
    torch.save({"logits": logits, "tokens": tokens, "stats": stats}, out)
model.model._closed = True
dist.barrier()
