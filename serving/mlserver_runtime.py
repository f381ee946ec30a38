"""MLServer runtime (reference: ``serving/mlserver/single-rank-mlmodel.py`` and ``multi-rank-mlmodel.py``): a
``MLModel`` that holds an ``AutoModel`` in-process (single rank) or forwards to the gRPC launcher (multi rank).
MLServer itself is optional: without it the class still works as a plain object (``load()`` / ``predict_ids()``)."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

try:                                       # pragma: no cover - optional dependency
    from mlserver import MLModel
    from mlserver.codecs import NumpyCodec
    from mlserver.types import InferenceResponse
    _HAVE = True
except Exception:                          # MLServer not installed: keep the runtime usable as a library
    MLModel = object
    _HAVE = False


class XFTRuntime(MLModel):
    def __init__(self, settings=None, model_path=None, dtype="bf16", grpc_target=None, **gen):
        if _HAVE and settings is not None:
            super().__init__(settings)
            extra = getattr(settings.parameters, "extra", {}) or {}
            model_path = model_path or settings.parameters.uri
            dtype = extra.get("dtype", dtype)
            grpc_target = extra.get("grpc_target", grpc_target)
            gen = {**extra.get("generate", {}), **gen}
        self.model_path, self.dtype, self.grpc_target, self.gen = model_path, dtype, grpc_target, gen
        self.model = self.client = None

    def load_sync(self) -> bool:
        if self.grpc_target:
            from serving.server import Client
            self.client = Client(self.grpc_target)
        else:
            import xfastertransformer_b200 as xft
            self.model = xft.AutoModel.from_pretrained(self.model_path, dtype=self.dtype)
        return True

    async def load(self) -> bool:
        return self.load_sync()

    def predict_ids(self, ids, **kw):
        import torch
        kw = {**self.gen, **kw}
        if self.client is not None:
            r = self.client.predict(ids, **kw)
            return torch.tensor(r["Ids"]).view(r["batch_size"], -1)
        return self.model.generate(torch.tensor(ids), **kw)

    async def predict(self, payload):      # pragma: no cover - needs MLServer
        arr = NumpyCodec.decode_input(payload.inputs[0])
        out = self.predict_ids(arr.tolist())
        return InferenceResponse(model_name=self.name, outputs=[NumpyCodec.encode_output("output_ids", out.numpy())])
