"""Hand-made GPTQ-converted checkpoint directories for tests: a synthetic Llama-style model whose five projections per
layer are replaced by per-channel codes + scales + zeros in the converter's on-disk layout."""
import configparser
import os

import numpy as np
import torch

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.tools.synthetic import write_synthetic_checkpoint


def make_gptq_dir(d: str, cfg, qt: str, seed: int = 0, std: float = 0.08) -> str:
    """qt: "int8" or "uint4".  Returns d; the dense fp32 twin is NOT kept (only the quantised tensors remain)."""
    write_synthetic_checkpoint(d, cfg, seed=seed, dtype="fp32", std=std)
    H, I = cfg.hidden_size, cfg.inter_size
    q_all = cfg.head_num * cfg.size_per_head + 2 * cfg.kv_head_num * cfg.size_per_head
    q_sz = cfg.head_num * cfg.size_per_head
    for i in range(cfg.num_layer):
        for name, (inf, outf) in {"attention.query_key_value": (H, q_all), "attention.dense": (q_sz, H),
                                  "mlp.gate_proj": (H, I), "mlp.up_proj": (H, I), "mlp.down_proj": (I, H)}.items():
            f = os.path.join(d, f"model.layers.{i}.{name}.weight.0.bin")
            w = torch.from_numpy(np.fromfile(f, dtype=np.float32).reshape(inf, outf)).t().contiguous()   # [out,in]
            if qt == "int8":
                q, s, z = R.quantize_int8_per_channel(w)
                q.t().contiguous().numpy().tofile(f.replace(".weight.0.bin", ".qweight.0.bin"))
            else:
                p, s, z = R.quantize_uint4_per_channel(w)
                qq = R.unpack_nibbles(p).t().contiguous()                    # [in, out], packed along out
                R.pack_nibbles(qq).numpy().tofile(f.replace(".weight.0.bin", ".qweight.0.bin"))
            s.numpy().tofile(f.replace(".weight.0.bin", ".scales.0.bin"))
            z.numpy().tofile(f.replace(".weight.0.bin", ".zeros.0.bin"))
            os.remove(f)
    cp = configparser.ConfigParser()
    cp.read(os.path.join(d, "config.ini"))
    cp[cfg.model_type].update({"quant_qweight_data_type": qt, "quant_scales_data_type": "fp32",
                               "quant_zeros_data_type": "fp32", "quant_groupsize": "-1"})
    with open(os.path.join(d, "config.ini"), "w") as fh:
        cp.write(fh)
    return d
