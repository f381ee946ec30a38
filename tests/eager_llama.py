"""Independent PyTorch-eager Llama (HF-style dense attention, no paging, no TP) that reads a
converted checkpoint directory.  The oracle for the end-to-end tests."""
import configparser
import math
import os

import numpy as np
import torch
import torch.nn.functional as F


def _load(path, name, shape, dtype):
    np_dt = {"fp32": np.float32, "fp16": np.float16, "bf16": np.uint16}[dtype]
    a = np.fromfile(os.path.join(path, name), dtype=np_dt).reshape(shape)
    t = torch.from_numpy(a.copy())
    if dtype == "bf16":
        t = t.view(torch.bfloat16)
    return t.float()


class EagerLlama:
    def __init__(self, path):
        cp = configparser.ConfigParser()
        cp.read(os.path.join(path, "config.ini"))
        c = cp[cp.sections()[0]]
        self.H = int(c["hidden_size"]); self.nh = int(c["head_num"]); self.nkv = int(c["kv_head_num"])
        self.D = int(c["size_per_head"]); self.I = int(c["inter_size"]); self.L = int(c["num_layer"])
        self.V = int(c["vocab_size"]); self.eps = float(c.get("layernorm_eps", 1e-6))
        self.theta = float(c.get("rope_theta", 10000)); dt = c["weight_data_type"]
        H, D = self.H, self.D
        q, kv = self.nh * D, self.nkv * D
        self.wte = _load(path, "model.wte.bin", (self.V, H), dt)
        self.fn = _load(path, "model.final_layernorm.weight.bin", (H,), dt)
        self.head = _load(path, "model.lm_head.weight.bin", (self.V, H), dt)
        self.layers = []
        for i in range(self.L):
            p = f"model.layers.{i}."
            self.layers.append(dict(
                n1=_load(path, p + "input_layernorm.weight.bin", (H,), dt),
                qkv=_load(path, p + "attention.query_key_value.weight.0.bin", (H, q + 2 * kv), dt),
                o=_load(path, p + "attention.dense.weight.0.bin", (q, H), dt),
                n2=_load(path, p + "post_attention_layernorm.weight.bin", (H,), dt),
                g=_load(path, p + "mlp.gate_proj.weight.0.bin", (H, self.I), dt),
                u=_load(path, p + "mlp.up_proj.weight.0.bin", (H, self.I), dt),
                d=_load(path, p + "mlp.down_proj.weight.0.bin", (self.I, H), dt)))

    def _norm(self, x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * w

    def _rope(self, x, pos):
        D = self.D
        inv = 1.0 / (self.theta ** (torch.arange(0, D, 2).float() / D))
        f = torch.outer(pos.float(), inv)
        cos, sin = f.cos()[None, :, None, :], f.sin()[None, :, None, :]
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    def logits(self, ids):
        """ids [B,S] -> fp32 logits [B,S,V] (full causal forward)."""
        B, S = ids.shape
        x = self.wte[ids]
        pos = torch.arange(S)
        mask = torch.full((S, S), float("-inf")).triu(1)
        g = self.nh // self.nkv
        for l in self.layers:
            h = self._norm(x, l["n1"])
            qkv = h @ l["qkv"]
            q = qkv[..., : self.nh * self.D].view(B, S, self.nh, self.D)
            k = qkv[..., self.nh * self.D:(self.nh + self.nkv) * self.D].view(B, S, self.nkv, self.D)
            v = qkv[..., (self.nh + self.nkv) * self.D:].view(B, S, self.nkv, self.D)
            q, k = self._rope(q, pos), self._rope(k, pos)
            k, v = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
            s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(self.D) + mask
            a = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v).reshape(B, S, -1)
            x = x + a @ l["o"]
            h = self._norm(x, l["n2"])
            x = x + (F.silu(h @ l["g"]) * (h @ l["u"])) @ l["d"]
        return self._norm(x, self.fn) @ self.head.t()

    def greedy(self, ids, new_tokens):
        ids = ids.clone()
        for _ in range(new_tokens):
            nxt = self.logits(ids)[:, -1].argmax(-1)
            ids = torch.cat([ids, nxt[:, None]], 1)
        return ids
