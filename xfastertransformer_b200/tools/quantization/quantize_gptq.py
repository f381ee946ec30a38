#!/usr/bin/env python
"""Per-channel GPTQ quantisation of a Llama-family HuggingFace checkpoint into the AutoGPTQ tensor layout, with nothing
but PyTorch — the artefact this repository ships in place of the reference's recipe, which patches the AutoGPTQ
package to run on CPUs (reference: tools/quantization/README.md, autogptq-cpu.patch) and needs AutoAWQ / AutoGPTQ
installed.  The output directory is what ``LlamaConvert().convert(dir, out, from_quantized_model="gptq")`` reads:
``*.qweight`` int32 packed along the input dimension, ``*.qzeros`` int32 holding zero - 1, ``*.scales`` fp16, and a
``quantization_config`` in ``config.json``.

    python -m xfastertransformer_b200.tools.quantization.quantize_gptq <hf_dir> <out_dir> --bits 4 \\
        [--calib text_file] [--samples 32] [--seq-len 512] [--device cuda] [--awq]

Algorithm (GPTQ, Frantar et al. 2022, per output channel = ``group_size -1``, asymmetric): for every linear layer the
inputs of a calibration run give H = 2 XᵀX / n; columns are quantised one by one in their natural order and the rounding
error of a column is spread over the columns not yet quantised through the Cholesky factor of H⁻¹, so that the layer's
OUTPUT error, not the weight error, is minimised.  Scales and zero points come from each output channel's min / max.
All layers are calibrated in one pass over the unquantised model (AutoGPTQ calibrates block by block on the already
quantised prefix; the difference is small at 8 bits and modest at 4).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict, Tuple

import torch


def quant_params(W: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel (row) scale and integer zero point of an asymmetric min / max grid."""
    qmax = (1 << bits) - 1
    lo = torch.minimum(W.min(1).values, torch.zeros(W.shape[0], device=W.device))
    hi = torch.maximum(W.max(1).values, torch.zeros(W.shape[0], device=W.device))
    scale = ((hi - lo) / qmax).clamp_min(1e-8)
    zero = torch.round(-lo / scale).clamp(0, qmax)
    return scale, zero


def rtn_quantize(W: torch.Tensor, bits: int):
    """Round to nearest on the same grid (the baseline GPTQ improves on)."""
    qmax = (1 << bits) - 1
    scale, zero = quant_params(W, bits)
    q = torch.clamp(torch.round(W / scale[:, None]) + zero[:, None], 0, qmax)
    return q.to(torch.int32), scale, zero.to(torch.int32)


def gptq_quantize(W: torch.Tensor, H: torch.Tensor, bits: int, damp: float = 0.01, block: int = 128):
    """W [out, in] fp32, H [in, in] = 2 XᵀX / n of the layer's inputs -> (q int32 [out, in], scale [out], zero int32 [out]).
    Dequantised weight = (q - zero) * scale."""
    W = W.clone().float()
    H = H.clone().float()
    n_in = W.shape[1]
    qmax = (1 << bits) - 1
    scale, zero = quant_params(W, bits)
    dead = torch.diag(H) == 0                     # inputs that never fired: any value is as good
    H[dead, dead] = 1.0
    W[:, dead] = 0.0
    H += torch.eye(n_in, device=H.device) * damp * torch.diag(H).mean()
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    Q = torch.zeros_like(W)
    for i0 in range(0, n_in, block):
        i1 = min(i0 + block, n_in)
        Wb = W[:, i0:i1].clone()
        Eb = torch.zeros_like(Wb)
        Hb = Hinv[i0:i1, i0:i1]
        for j in range(i1 - i0):
            w = Wb[:, j]
            q = torch.clamp(torch.round(w / scale) + zero, 0, qmax)
            Q[:, i0 + j] = q
            err = (w - (q - zero) * scale) / Hb[j, j]
            Wb[:, j:] -= err[:, None] * Hb[j, j:][None, :]
            Eb[:, j] = err
        W[:, i1:] -= Eb @ Hinv[i0:i1, i1:]
    return Q.to(torch.int32), scale, zero.to(torch.int32)


def awq_search_scale(weights, H: torch.Tensor, x_absmean: torch.Tensor, bits: int, grid: int = 20):
    """Activation-aware scaling (AWQ, Lin et al. 2023) for linear layers that share one input: find per-input-channel
    factors s so that quantising W * s and feeding x / s loses the least OUTPUT — channels with large activations get
    their weight columns enlarged and so keep more of the grid.  s = mean|x|^ratio, normalised to sqrt(max * min) = 1,
    ratio searched over `grid` values in [0, 1); the loss of a candidate is sum over the layers of tr(D H D^T) with
    D = W - Q(W s) / s and H = X^T X of the shared input, so no activations need to be kept.  Returns (s [in], ratio,
    loss at ratio, loss without scaling)."""
    H = H.float()
    xm = x_absmean.float().clamp_min(1e-8)

    def loss_for(s):
        tot = 0.0
        for W in weights:
            Wf = W.float()
            q, sc, z = rtn_quantize(Wf * s[None, :], bits)
            D = Wf - ((q - z[:, None]).float() * sc[:, None]) / s[None, :]
            tot += float(((D @ H) * D).sum())
        return tot

    ones = torch.ones_like(xm)
    base = loss_for(ones)
    best = (ones, 0.0, base)
    for i in range(1, grid):
        ratio = i / grid
        s = xm.pow(ratio).clamp_min(1e-4)
        s = s / (s.max() * s.min()).sqrt()
        l = loss_for(s)
        if l < best[2]:
            best = (s, ratio, l)
    return best[0], best[1], best[2], base


def pack_autogptq(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, bits: int) -> Dict[str, torch.Tensor]:
    """[out, in] levels -> AutoGPTQ tensors: qweight int32 [in / pack, out], qzeros int32 [1, out / pack] holding
    zero - 1 (modulo 2^bits), scales fp16 [1, out], g_idx zeros."""
    import numpy as np
    pack, qmax = 32 // bits, (1 << bits) - 1
    out_f, in_f = q.shape
    if in_f % pack or out_f % pack:
        raise ValueError(f"dimensions {out_f} x {in_f} must be multiples of {pack} for {bits}-bit packing")
    qt = q.t().contiguous().to(torch.int64).view(in_f // pack, pack, out_f)
    qweight = sum(qt[:, j, :] << (bits * j) for j in range(pack))
    zs = ((zero.to(torch.int64) - 1) & qmax).view(1, out_f // pack, pack)
    qzeros = sum(zs[:, :, j] << (bits * j) for j in range(pack))
    to_i32 = lambda t: torch.from_numpy(t.cpu().numpy().astype(np.uint32).view(np.int32).copy())
    return {"qweight": to_i32(qweight), "qzeros": to_i32(qzeros), "scales": scale.view(1, -1).half().cpu(),
            "g_idx": torch.zeros(in_f, dtype=torch.int32)}


def calibrate(model, batches, device="cpu"):
    """One pass of the calibration batches through the unquantised model.  Returns, per decoder linear (by module name):
    the module, sum of 2 x^T x, sum of |x| per input channel, number of rows seen."""
    targets = {name: mod for name, mod in model.named_modules()
               if isinstance(mod, torch.nn.Linear) and ".layers." in name and name.endswith("_proj")}
    hess = {name: torch.zeros(m.in_features, m.in_features, device=device) for name, m in targets.items()}
    absmean = {name: torch.zeros(m.in_features, device=device) for name, m in targets.items()}
    count = {name: 0 for name in targets}

    def hook(name):
        def fn(_, inp):
            x = inp[0].detach().reshape(-1, inp[0].shape[-1]).float()
            hess[name] += 2.0 * (x.t() @ x)
            absmean[name] += x.abs().sum(0)
            count[name] += x.shape[0]
        return fn
    handles = [m.register_forward_pre_hook(hook(n)) for n, m in targets.items()]
    with torch.no_grad():
        for b in batches:
            model(b.to(device))
    for h in handles:
        h.remove()
    return targets, hess, absmean, count


def apply_awq(model, batches, bits: int = 4, device="cpu"):
    """Calibrate and fold activation-aware scales into `model` in place (same function, friendlier weights); returns
    the statistics of the SCALED model for a following `gptq_quantize`."""
    targets, hess, absmean, count = calibrate(model, batches, device)
    _apply_awq(model, targets, hess, absmean, count, bits)
    return targets, hess, absmean, count


def quantize_checkpoint(hf_dir: str, out_dir: str, bits: int = 4, calib: str = "", samples: int = 32, seq_len: int = 512,
                        device: str = "cpu", seed: int = 0, awq: bool = False) -> str:
    """Quantise every decoder linear of the HF causal LM in `hf_dir` and write an AutoGPTQ-format directory.  With
    `awq`, an activation-aware scale search runs first (the reference's recipe puts AutoAWQ with `export_compatible` in
    front of AutoGPTQ): the factors are folded into the weights and into whatever produces their input — the norm gain
    for q / k / v and gate / up, the rows of up_proj for down_proj, the rows of v_proj for o_proj when their sizes match —
    so the written model computes the same function before rounding and is an ordinary GPTQ checkpoint after it."""
    from safetensors.torch import save_file
    from transformers import AutoConfig, AutoModelForCausalLM
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    cfg = AutoConfig.from_pretrained(hf_dir)
    model = AutoModelForCausalLM.from_pretrained(hf_dir, torch_dtype=torch.float32).to(device).eval()
    g = torch.Generator().manual_seed(seed)
    if calib:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(hf_dir)
        ids = tok(open(calib).read(), return_tensors="pt").input_ids[0]
        n = max(1, min(samples, ids.numel() // seq_len))
        batches = [ids[i * seq_len:(i + 1) * seq_len][None] for i in range(n)]
    else:
        # no text given: uniformly random token ids still exercise every input direction of every layer
        batches = [torch.randint(0, cfg.vocab_size, (1, seq_len), generator=g) for _ in range(samples)]
    targets, hess, absmean, count = calibrate(model, batches, device)
    if awq:
        _apply_awq(model, targets, hess, absmean, count, bits)
    tensors = {}
    for name, p in model.state_dict().items():
        base = name[: -len(".weight")] if name.endswith(".weight") else None
        if base in targets:
            q, s, z = gptq_quantize(p.float(), hess[base] / max(count[base], 1), bits)
            for k, v in pack_autogptq(q, s, z, bits).items():
                tensors[f"{base}.{k}"] = v
        else:
            tensors[name] = p.detach().cpu().contiguous()
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    conf = cfg.to_dict()
    conf["quantization_config"] = {"quant_method": "gptq", "bits": bits, "group_size": -1, "sym": False, "desc_act": False}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(conf, f, indent=1)
    for extra in ("tokenizer.model", "tokenizer.json", "tokenizer_config.json", "special_tokens_map.json",
                  "generation_config.json"):
        if os.path.exists(os.path.join(hf_dir, extra)):
            shutil.copy(os.path.join(hf_dir, extra), os.path.join(out_dir, extra))
    return out_dir


def _apply_awq(model, targets, hess, absmean, count, bits) -> None:
    """Scale search per decoder layer and group of linears with a common input; weights, producers of their inputs and
    the collected statistics are rewritten in place (x -> x / s turns H into diag(1/s) H diag(1/s))."""
    by_layer: Dict[str, Dict[str, str]] = {}
    for name in targets:
        prefix, leaf = name.rsplit(".", 1)
        layer = prefix.rsplit(".", 1)[0]                  # "...layers.N"
        by_layer.setdefault(layer, {})[leaf] = name
    mods = dict(model.named_modules())

    def rescale_stats(names, s):
        for n in names:
            hess[n] = hess[n] / s[:, None] / s[None, :]
            absmean[n] = absmean[n] / s

    with torch.no_grad():
        for layer, leaves in by_layer.items():
            groups = []
            if all(k in leaves for k in ("q_proj", "k_proj", "v_proj")) and (layer + ".input_layernorm") in mods:
                groups.append((["q_proj", "k_proj", "v_proj"], ("norm", mods[layer + ".input_layernorm"])))
            if "o_proj" in leaves and "v_proj" in leaves and \
                    targets[leaves["v_proj"]].out_features == targets[leaves["o_proj"]].in_features:
                groups.append((["o_proj"], ("rows", targets[leaves["v_proj"]])))
            if all(k in leaves for k in ("gate_proj", "up_proj")) and (layer + ".post_attention_layernorm") in mods:
                groups.append((["gate_proj", "up_proj"], ("norm", mods[layer + ".post_attention_layernorm"])))
            if "down_proj" in leaves and "up_proj" in leaves:
                groups.append((["down_proj"], ("rows", targets[leaves["up_proj"]])))
            for members, (kind, producer) in groups:
                names = [leaves[m] for m in members]
                n0 = names[0]
                H = hess[n0] / max(count[n0], 1)
                s, ratio, _, _ = awq_search_scale([targets[n].weight.data for n in names], H,
                                                  absmean[n0] / max(count[n0], 1), bits)
                if ratio == 0.0:
                    continue
                for n in names:
                    targets[n].weight.data = (targets[n].weight.data.float() * s[None, :]).to(targets[n].weight.dtype)
                if kind == "norm":
                    producer.weight.data = (producer.weight.data.float() / s).to(producer.weight.dtype)
                    if getattr(producer, "bias", None) is not None:
                        producer.bias.data = (producer.bias.data.float() / s).to(producer.bias.dtype)
                else:
                    producer.weight.data = (producer.weight.data.float() / s[:, None]).to(producer.weight.dtype)
                    if producer.bias is not None:
                        producer.bias.data = (producer.bias.data.float() / s).to(producer.bias.dtype)
                rescale_stats(names, s)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("hf_dir")
    ap.add_argument("out_dir")
    ap.add_argument("--bits", type=int, default=4, choices=(4, 8))
    ap.add_argument("--calib", default="", help="text file with calibration text (default: random token ids)")
    ap.add_argument("--samples", type=int, default=32)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--awq", action="store_true", help="activation-aware scale search before GPTQ (the AutoAWQ step of the reference's recipe)")
    a = ap.parse_args()
    print(quantize_checkpoint(a.hf_dir, a.out_dir, a.bits, a.calib, a.samples, a.seq_len, a.device, awq=a.awq))


if __name__ == "__main__":
    main()
