"""Stateful layer-level C++ API (csrc/core/layer_objects.cc) driven through its C wrappers: a whole Llama layer with
its own KV cache (prefill, then decode steps) and the DeepSeek MoE object (bf16 and fp8 block-scaled experts),
against the pure-PyTorch reference ops."""
import ctypes as C
import math
import os

import pytest
import torch

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.runtime.loader import make_linear

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _core():
    lib = C.CDLL(os.path.join(ROOT, "xfastertransformer_b200", "lib", "libxft_b200_core.so"))
    lib.xftc_dsmoe_create.restype = C.c_void_p
    lib.xftc_dsmoe_create.argtypes = [C.c_int] * 7 + [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_float]
    lib.xftc_dsmoe_forward_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.xftc_dsmoe_forward_selected.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    lib.xftc_dsmoe_destroy.argtypes = [C.c_void_p]
    lib.xftc_layer_llama.argtypes = [C.c_int] * 9 + [C.c_void_p] * 11
    lib.xftc_attention_llama.argtypes = [C.c_int] * 8 + [C.c_void_p] * 6
    return lib


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _ref_layer(x, past_k, past_v, w, heads, kv_heads, D, pos0):
    """fp32 reference of one pre-norm Llama layer on [B, S, H] with an explicit KV history."""
    B, S, H = x.shape
    h = R.rmsnorm(x, w["ln1"], 1e-6)
    q = (h @ w["q"]).view(B, S, heads, D)
    k = (h @ w["k"]).view(B, S, kv_heads, D)
    v = (h @ w["v"]).view(B, S, kv_heads, D)
    table = R.rope_table(pos0 + S, D, 10000.0)
    pos = torch.arange(pos0, pos0 + S)
    outs = []
    for b in range(B):
        qb, kb = R.rope_apply(q[b], k[b], pos, table, D, "half")
        ks = torch.cat([past_k[b], kb], 0)
        vs = torch.cat([past_v[b], v[b]], 0)
        past_k[b], past_v[b] = ks, vs
        g = heads // kv_heads
        o = torch.empty(S, heads, D)
        for hh in range(heads):
            sc = (qb[:, hh] @ ks[:, hh // g].t()) / math.sqrt(D)
            mask = torch.arange(ks.shape[0])[None, :] > (pos0 + torch.arange(S))[:, None]
            sc = sc.masked_fill(mask, float("-inf"))
            o[:, hh] = torch.softmax(sc, -1) @ vs[:, hh // g]
        outs.append(o.reshape(S, heads * D))
    a = torch.stack(outs)
    x1 = x + a @ w["o"]
    h2 = R.rmsnorm(x1, w["ln2"], 1e-6)
    return x1 + (torch.nn.functional.silu(h2 @ w["gate"]) * (h2 @ w["up"])) @ w["down"]


def test_invoke_layer_llama_prefill_then_decode():
    lib = _core()
    g = torch.Generator().manual_seed(0)
    B, S, H, heads, kvh, D, I, max_pos = 2, 70, 256, 4, 2, 64, 704, 256
    bf = lambda *s, std=0.05: (torch.randn(*s, generator=g) * std).bfloat16()
    w16 = dict(q=bf(H, heads * D), k=bf(H, kvh * D), v=bf(H, kvh * D), o=bf(heads * D, H), gate=bf(H, I), up=bf(H, I),
               down=bf(I, H))
    ln1 = 1 + 0.1 * torch.randn(H, generator=g)
    ln2 = 1 + 0.1 * torch.randn(H, generator=g)
    wref = {k: v.float() for k, v in w16.items()}
    wref.update(ln1=ln1, ln2=ln2)
    dev = {k: v.cuda() for k, v in w16.items()}
    ln1d, ln2d = ln1.cuda(), ln2.cuda()
    past_k = [torch.empty(0, kvh, D) for _ in range(B)]
    past_v = [torch.empty(0, kvh, D) for _ in range(B)]
    pos0 = 0
    for step, seq in enumerate([S, 1, 1, 1]):
        x = bf(B, seq, H, std=1.0)
        want = _ref_layer(x.float(), past_k, past_v, wref, heads, kvh, D, pos0)
        xd = x.cuda().view(B * seq, H)
        out = torch.empty_like(xd)
        rc = lib.xftc_layer_llama(B, seq, D, heads, kvh, max_pos, pos0, H, I, _p(out), _p(xd), _p(ln1d), _p(dev["q"]),
                                  _p(dev["k"]), _p(dev["v"]), _p(dev["o"]), _p(ln2d), _p(dev["gate"]), _p(dev["up"]),
                                  _p(dev["down"]))
        assert rc == 0, rc
        torch.cuda.synchronize()
        err = (out.float().cpu().view(B, seq, H) - want).abs().max().item()
        assert err < 0.06 * max(1.0, want.abs().max().item()), (step, err)
        pos0 += seq


@pytest.mark.parametrize("fp8", [False, True])
def test_deepseek_moe_object(fp8):
    lib = _core()
    g = torch.Generator().manual_seed(3)
    T, E, k, H, I, ng, tg = 37, 16, 4, 256, 128, 4, 2
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    gu = torch.randn(E, 2 * I, H, generator=g) * 0.05
    dn = torch.randn(E, H, I, generator=g) * 0.05
    bias = torch.randn(E, generator=g) * 0.1
    logits = torch.randn(T, E, generator=g)
    if fp8:
        def q(w):      # [E, rows, cols] -> e4m3 bytes + scales [E, rows/128, cols/128]; returns the dequantised copy too
            Ee, r, c = w.shape
            blocks = w.view(Ee, r // 128, 128, c // 128, 128)
            sc = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-8) / 448.0
            qv = (blocks / sc[:, :, None, :, None]).to(torch.float8_e4m3fn)
            deq = (qv.float() * sc[:, :, None, :, None]).view(Ee, r, c)
            return qv.view(Ee, r, c).view(torch.uint8), sc.contiguous(), deq
        guq, gus, gu = q(gu)
        dnq, dns, dn = q(dn)
        args_w = (guq.cuda(), dnq.cuda(), gus.cuda(), dns.cuda())
    else:
        gu, dn = gu.bfloat16().float(), dn.bfloat16().float()
        args_w = (gu.bfloat16().cuda(), dn.bfloat16().cuda(), None, None)
    experts = [(make_linear(gu[e], "bf16"), make_linear(dn[e], "bf16")) for e in range(E)]
    idx, w = R.route_deepseek(logits, bias, k, ng, tg, 2.5, True, "sigmoid")
    want = R.moe_experts(x.float(), idx, w, experts, "silu")
    biasd, xd, logd = bias.cuda(), x.cuda(), logits.cuda()
    moe = lib.xftc_dsmoe_create(E, k, H, I, 1, ng, tg, _p(args_w[0]), _p(args_w[1]), _p(args_w[2]), _p(args_w[3]), _p(biasd),
                                128, 0, 1, 2.5)
    assert moe
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    assert lib.xftc_dsmoe_forward_logits(moe, _p(xd), _p(out), T, _p(logd)) == 0
    torch.cuda.synchronize()
    err = (out.float().cpu() - want).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err
    # pre-selected experts give the same answer
    out2 = torch.empty_like(out)
    idxd, wd = idx.int().cuda(), w.float().cuda()
    assert lib.xftc_dsmoe_forward_selected(moe, _p(xd), _p(out2), T, _p(idxd), _p(wd)) == 0
    torch.cuda.synchronize()
    assert (out2.float() - out.float()).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
    lib.xftc_dsmoe_destroy(moe)


_KEEP = []


@pytest.mark.parametrize("routed,shared", [(16, 1), (16, 0), (0, 0)])
def test_invoke_moe_deepseek_stateless(routed, shared):
    """invokeMoEDeepSeek: one weight set for every routed expert and the shared expert, DeepSeek-V3 routing constants
    (include/layers_mlp.h:25 of the reference); routed == 0 is the dense layer."""
    lib = _core()
    lib.xftc_invoke_moe_deepseek.restype = C.c_int
    g = torch.Generator().manual_seed(routed + shared)
    T, H, I, MI = 21, 256, 384, 128
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    inter = MI if routed else I
    gate = (torch.randn(H, inter, generator=g) * 0.05).bfloat16()          # [in, out], as the reference passes them
    up = (torch.randn(H, inter, generator=g) * 0.05).bfloat16()
    down = (torch.randn(inter, H, generator=g) * 0.05).bfloat16()
    gw = torch.randn(H, max(routed, 1), generator=g) * 0.3
    gb = torch.randn(max(routed, 1), generator=g) * 0.1
    mlp = lambda v: (torch.nn.functional.silu(v @ gate.float()) * (v @ up.float())).bfloat16().float() @ down.float()
    xf = x.float()
    if routed:
        logits = xf @ gw.bfloat16().float()
        idx, w = R.route_deepseek(logits, gb, 8, 8, 4, 2.5, True, "sigmoid")
        want = w.sum(-1, keepdim=True) * mlp(xf)
        if shared:
            want = want + mlp(xf)
    else:
        want = mlp(xf)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    dev = [t.cuda() for t in (x, gw, gb, gate, up, down)]
    _KEEP.append(dev)       # the entry point keeps [out, in] copies per weight ADDRESS: the weights must stay where they are
    rc = lib.xftc_invoke_moe_deepseek(T, H, I, MI, shared, routed, _p(out), _p(dev[0]), _p(dev[1]), _p(dev[2]), _p(dev[3]),
                                      _p(dev[4]), _p(dev[5]))
    assert rc == 0, rc
    torch.cuda.synchronize()
    err = (out.float().cpu() - want).abs().max().item()
    assert err < 3e-2 * max(1.0, want.abs().max().item()), err
