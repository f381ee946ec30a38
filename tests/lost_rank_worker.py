"""torchrun worker for the lost-rank test: rank 1 leaves between two requests (no collective in flight); rank 0's next
request must end with CommError within the process-group time-out instead of hanging."""
import sys
import time

import torch

import xfastertransformer_b200 as xft
from xfastertransformer_b200.parallel.dist import CommError

path, out = sys.argv[1], sys.argv[2]
model = xft.AutoModel.from_pretrained(path, dtype="bf16")
ids = torch.randint(0, 32000, (1, 8), generator=torch.Generator().manual_seed(1))
if model.rank == 0:
    first = model.generate(ids, max_length=12)
    time.sleep(1.0)                      # rank 1 is gone by now
    t0 = time.time()
    try:
        model.generate(ids, max_length=12)
        res = "no error"
    except CommError as e:
        res = "CommError"
    except Exception as e:               # anything else is reported, the test decides
        res = f"{type(e).__name__}: {e}"
    with open(out, "w") as f:
        f.write(f"{res}\n{time.time() - t0:.2f}\n{first.shape[1]}\n")
    model.model._closed = True
else:
    model.generate()                     # serve exactly one request, then leave without a word
    sys.exit(0)
