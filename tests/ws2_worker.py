"""torchrun worker for test_ws2_gloo: rank 0 drives, rank 1 follows."""
import sys

import torch
import torch.distributed as dist

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
g = torch.Generator().manual_seed(1)
ids = torch.randint(0, 32000, (2, 32), generator=g)
m = model.model
if model.rank == 0:
    sid = model.set_input_cb(ids.tolist(), None, 64)
    logits = model.forward_cb()
    model.free_seqs(sid)
    tokens = model.generate(ids, max_length=48)
else:
    # followers ignore their arguments and execute what rank 0 broadcasts
    model.set_input_cb()
    model.forward_cb()
    model.free_seqs()
    model.generate()
ffn = [None, None]
dist.all_gather_object(ffn, m.decoder.layers[0].down.in_features)
if model.rank == 0:
    torch.save({"logits": logits, "tokens": tokens, "ffn": ffn, "all_reduce": m.ctx.stats["all_reduce"],
                "pairs": m.prefill_decoder.pairs_run}, out)
m._closed = True
dist.barrier()
