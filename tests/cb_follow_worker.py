"""torchrun worker: rank 0 drives a continuous-batching session (greedy fast path and logits path), the other ranks sit
in follow_cb() until rank 0 shuts them down."""
import sys

import torch

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
if model.rank != 0:
    model.follow_cb()
    sys.exit(0)
g = torch.Generator().manual_seed(1)
ids = torch.randint(0, 32000, (2, 32), generator=g)
sids = model.set_input_cb(ids.tolist(), None, 64, greedy=True)
toks = [model.forward_cb_greedy()]
for _ in range(5):
    model.set_input_cb([[int(t)] for t in toks[-1]], sids, None, greedy=True)
    toks.append(model.forward_cb_greedy())
# one step through the logits path in the same session
model.set_input_cb([[int(t)] for t in toks[-1]], sids, None)
logits = model.forward_cb()
toks.append(logits.argmax(-1))
model.free_seqs(sids)
torch.save({"tokens": torch.stack(toks, 1)}, out)
model.model.exit_slaves()
