"""torchrun worker: the non-zero ranks sit in model.follow() while rank 0 uses, in turn, generate (greedy and beams),
config + input + forward step by step, the continuous-batching calls and all-position logits; then it shuts them down."""
import sys

import torch

import xfastertransformer_b200 as xft

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
if model.rank != 0:
    model.follow()
    sys.exit(0)
g = torch.Generator().manual_seed(1)
ids = torch.randint(0, 32000, (2, 32), generator=g)
res = {"greedy": model.generate(ids, max_length=40)}
res["beams"] = model.generate(ids[:, :12], max_length=18, num_beams=2)
model.config(max_length=36)
model.input(ids)
steps = []
while not model.is_done():
    steps.append(model.forward())
res["stepwise"] = model.finalize()
sids = model.set_input_cb(ids.tolist(), None, 64)
res["cb_logits"] = model.forward_cb()
model.free_seqs(sids)
res["all"] = model(ids[:, :16])
torch.save(res, out)
model.model.exit_slaves()
