"""The decoder harness that bench.py times, against the oracle, layer by layer.

A 2-layer decoder with the full Llama-3-8B widths (hidden 4096, 32 q / 8 kv heads of 128, FFN 14336) runs 2 x 128 tokens
through ``W8A8Decoder.forward`` -- the very code path of the benchmark's one-GPU step -- with tracing on.  For every one of
the 14 Linears the traced input row is handed to the oracle's restatement of QLinearINT8Deploy.forward
(fms_mo/modules/linear.py:1309-1338, :1115-1188): int8 codes, per-token scales, int32 accumulators and the bf16 output
must equal the kernels' bit for bit.  The plumbing between the Linears (residual add, RMSNorm, RoPE, attention, SiLU * up)
is compared with plain PyTorch in fp32 to a stated tolerance, and the final hidden state with a free-running oracle chain.
"""

import pytest
import torch
import torch.nn.functional as F

from fms_model_optimizer_b200 import ops
from fms_model_optimizer_b200.decoder import LLAMA3_8B, W8A8Decoder
from oracle import qlinear as OL
from oracle import quantizers as OQ

pytestmark = pytest.mark.gpu

BF16_ULP = 2.0**-7  # relative spacing of bf16 values (one place of an 8-bit significand)


def _oracle_linear(lin, h):
    """QLinearINT8Deploy.forward on CPU for one of the decoder's Linears: (out bf16, codes, scale, int32 acc)."""
    st = OL.DeployState(lin.weight.cpu(), lin.w_scale.cpu().to(lin.w_scale_dtype), lin.smooth.cpu().bfloat16().reshape(1, -1),
                        torch.zeros(lin.weight.shape[0], dtype=torch.bfloat16), torch.tensor(127, dtype=torch.int), None)  # fmt: skip
    x2 = h / st.smoothq_scale
    codes, input_scale = OQ.qa_dynamic_max_qfunc(x2)
    acc = (codes.double() @ st.weight.double().t()).to(torch.int32)  # exact: |acc| < 2^53
    out = (acc.float() * (input_scale * st.w_scale).to(torch.float16) + st.bias).to(torch.float16).to(torch.bfloat16)
    return out, codes, input_scale.reshape(-1).float(), acc


def _close_bf16(got, want_f32, places=1.0, floor=1e-3):
    """|got - want| <= places bf16 places of max(|want|, floor)."""
    err = (got.float() - want_f32).abs()
    return bool((err <= places * BF16_ULP * want_f32.abs().clamp(min=floor)).all())


def _rope_ref(x, cos, sin, S):
    T, H, D = x.shape
    pos = torch.arange(T) % S
    c, s = cos[pos][:, None, :], sin[pos][:, None, :]
    a, b = x[..., : D // 2].float(), x[..., D // 2 :].float()
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def test_two_layer_decoder_every_linear_bit_exact_against_oracle(cuda_dev):
    cfg = dict(LLAMA3_8B, layers=2, batch=2, seq=128, vocab=4096)
    model = W8A8Decoder(cfg, cuda_dev, layers=2)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"]), generator=g).to(cuda_dev)
    model.trace = []
    out = model.forward(ids)
    torch.cuda.synchronize()
    ops.check_status(cuda_dev)
    tr = {(tag, li): t.cpu() for tag, li, t in model.trace}
    B, S, hd = cfg["batch"], cfg["seq"], cfg["head_dim"]
    T = B * S
    cos, sin = model.cos.cpu(), model.sin.cpu()
    x_chain = F.embedding(ids.cpu(), model.embed.cpu()).view(T, -1)  # free-running oracle chain of the residual stream
    pending_chain = None
    for li, lin in enumerate(model.layers):
        # ---- residual add + RMSNorm (plumbing): exact add, norm within one bf16 place of the fp32 formula
        x1 = tr[("x_attn_in", li)]
        if li == 0:
            assert torch.equal(x1, x_chain)
        h = tr[("h_attn", li)]
        assert _close_bf16(h, F.rms_norm(x1.float(), (x1.shape[-1],), None, 1e-5)), ("h_attn", li)
        # ---- q, k, v: codes, scales, accumulators, outputs bit for bit, from the row the kernels saw
        for name in "qkv":
            want, codes, scale, acc = _oracle_linear(lin[name], h)
            assert torch.equal(tr[("codes_" + name, li)], codes), (name, li)
            assert torch.equal(tr[("scale_" + name, li)], scale), (name, li)
            assert torch.equal(ops.imatmul(tr[("codes_" + name, li)].to(cuda_dev), lin[name].weight.t()).cpu(), acc), (name, li)
            assert torch.equal(tr[(name, li)], want), (name, li)
        # ---- RoPE and attention (plumbing)
        q, k, v = tr[("q", li)], tr[("k", li)], tr[("v", li)]
        qr, kr = tr[("q_rope", li)], tr[("k_rope", li)]
        assert _close_bf16(qr, _rope_ref(q.view(T, -1, hd), cos, sin, S)), ("rope q", li)
        assert _close_bf16(kr, _rope_ref(k.view(T, -1, hd), cos, sin, S)), ("rope k", li)
        a_ref = F.scaled_dot_product_attention(qr.view(B, S, -1, hd).transpose(1, 2).float(), kr.view(B, S, -1, hd).transpose(1, 2).float(),
                                               v.view(B, S, -1, hd).transpose(1, 2).float(), is_causal=True, enable_gqa=True)  # fmt: skip
        a = tr[("attn", li)]
        a_ref = a_ref.transpose(1, 2).reshape(T, -1)
        assert (a.float() - a_ref).abs().max() < 2e-2 * a_ref.abs().max(), ("attention", li)
        # ---- o
        want, codes, scale, acc = _oracle_linear(lin["o"], a)
        assert torch.equal(tr[("codes_o", li)], codes) and torch.equal(tr[("scale_o", li)], scale), ("o", li)
        assert torch.equal(tr[("o", li)], want), ("o", li)
        # ---- residual add + RMSNorm
        x2 = tr[("x_mlp_in", li)]
        assert torch.equal(x2, (x1.float() + tr[("o", li)].float()).bfloat16()), ("x += o", li)
        h2 = tr[("h_mlp", li)]
        assert _close_bf16(h2, F.rms_norm(x2.float(), (x2.shape[-1],), None, 1e-5)), ("h_mlp", li)
        for name in ("gate", "up"):
            want, codes, scale, acc = _oracle_linear(lin[name], h2)
            assert torch.equal(tr[("codes_" + name, li)], codes) and torch.equal(tr[("scale_" + name, li)], scale), (name, li)
            assert torch.equal(tr[(name, li)], want), (name, li)
        # ---- SiLU * up (plumbing) and down
        gt, u = tr[("gate", li)], tr[("up", li)]
        hd_ = tr[("h_down", li)]
        assert _close_bf16(hd_, F.silu(gt.float()).bfloat16().float() * u.float(), places=2.0, floor=1e-6), ("silu*up", li)
        want, codes, scale, acc = _oracle_linear(lin["down"], hd_)
        assert torch.equal(tr[("codes_down", li)], codes) and torch.equal(tr[("scale_down", li)], scale), ("down", li)
        assert torch.equal(ops.imatmul(tr[("codes_down", li)].to(cuda_dev), lin["down"].weight.t()).cpu(), acc), ("down acc", li)
        assert torch.equal(tr[("down", li)], want), ("down", li)

        # ---- the same layer free-running on the CPU (its own norms, rope, attention, SiLU): hidden states stay close
        if pending_chain is not None:
            x_chain = (x_chain.float() + pending_chain.float()).bfloat16()
        hc = F.rms_norm(x_chain.float(), (x_chain.shape[-1],), None, 1e-5).bfloat16()
        qc, kc, vc = (_oracle_linear(lin[n], hc)[0] for n in "qkv")
        qc = _rope_ref(qc.view(T, -1, hd), cos, sin, S).bfloat16()
        kc = _rope_ref(kc.view(T, -1, hd), cos, sin, S).bfloat16()
        ac = F.scaled_dot_product_attention(qc.view(B, S, -1, hd).transpose(1, 2).float(), kc.view(B, S, -1, hd).transpose(1, 2).float(),
                                            vc.view(B, S, -1, hd).transpose(1, 2).float(), is_causal=True, enable_gqa=True)  # fmt: skip
        oc = _oracle_linear(lin["o"], ac.transpose(1, 2).reshape(T, -1).bfloat16())[0]
        x_chain = (x_chain.float() + oc.float()).bfloat16()
        hc = F.rms_norm(x_chain.float(), (x_chain.shape[-1],), None, 1e-5).bfloat16()
        gc, uc = _oracle_linear(lin["gate"], hc)[0], _oracle_linear(lin["up"], hc)[0]
        pending_chain = _oracle_linear(lin["down"], (F.silu(gc.float()).bfloat16().float() * uc.float()).bfloat16())[0]
        got_x = (x2.float() + 0)  # residual stream after attention, as traced
        rel = ((got_x - x_chain.float()).norm() / x_chain.float().norm()).item()
        # the chain runs its own fp32 attention, norms and SiLU; a last-place difference in a normalised row flips int8
        # codes, and with random weights those flips are not damped from layer to layer (4 % measured after two layers)
        assert rel < 0.1, ("free-running chain", li, rel)
    assert out.shape == (B,)


def test_module_surface_close_to_fused_surface(cuda_dev):
    """The same 2-layer decoder built from QLinear -> lower_qmodel_b200 -> QLinearINT8Deploy modules (PyTorch norms and
    activations) against the fused path: same weights and codes up to the last place of the normalised rows."""
    cfg = dict(LLAMA3_8B, layers=2, batch=2, seq=128, vocab=2048, hidden=1024, q_heads=8, kv_heads=2, ffn=2816)
    ids = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"]), generator=torch.Generator().manual_seed(1)).to(cuda_dev)
    fused = W8A8Decoder(cfg, cuda_dev, layers=2)
    mods = W8A8Decoder(cfg, cuda_dev, layers=2, surface="modules")
    for li in range(2):
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            # the module route latches its weight clip values in a training-mode forward of QLinear, whose SmoothQuant
            # scale is formed with a scalar exponent (fms_mo/modules/linear.py:345-368), the fused route with the tensor
            # exponent of from_fms_mo (:799-817): rows where the two disagree in the last bf16 place get another scale
            wm, wf = mods.layers[li][name].weight, fused.layers[li][name].weight
            assert (wm != wf).float().mean().item() < 5e-3, (li, name, (wm != wf).float().mean().item())
            sm_, sf = mods.layers[li][name].w_scale.float().reshape(-1), fused.layers[li][name].w_scale
            assert ((sm_ - sf).abs() <= 2.0**-7 * sf.abs()).all(), (li, name)
    fused.forward(ids)
    hf = fused.last_hidden.float().clone()
    mods.forward(ids)
    hm = mods.last_hidden.float()
    rel = ((hf - hm).norm() / hm.norm()).item()
    assert rel < 2e-2, rel
