"""The QAT workload against the reference's own numbers: a two-layer BERT encoder with BERT-base widths whose twelve
Linears are this package's ``QLinear`` (PACT+ activations, clip values +-6, SAWB+ per-channel weights), one training-mode
forward and backward in fp32 with the loss ``(out * G).sum()``.

The golden file was produced by fms-model-optimizer itself on CPU (``qmodel_prep`` with the ``qat_int8`` recipe,
tests/golden/make_golden.py::gen_c4).  This test rebuilds the same random-init model from the same seed, swaps in this
package's QLinear at the module names the reference quantised, runs the step on the GPU and compares the output, every
clip-value gradient, every bias gradient and the sampled statistics of every weight gradient.

Tolerances.  The quantizer kernels are bit exact given their inputs (tests/test_gpu_quant.py).  What differs from the CPU
run is the order of fp32 sums: in the GEMMs, in LayerNorm / softmax, and in the row statistics behind the SAWB clip
values, which therefore agree only to a few fp32 places (3e-6 relative measured; asserted < 1e-4).  A clip value that
moves in its last places moves the rounding boundaries of a whole weight row, and a weight that crosses one changes by a
full quantisation level.  Measured on the reference itself, on CPU: multiplying every SAWB clip value of this model by
1 + 3e-6 * N(0, 1) changes the output by 1.4e-2 relative Frobenius (this kernel path: 1.15e-2).  The bounds below are
that figure with head-room, not a statement about the kernels' accuracy: 3e-2 on the output, 5e-2 on gradients.
"""

import pytest
import torch

from conftest import load_golden
from fms_model_optimizer_b200 import ops
from fms_model_optimizer_b200.modules import QLinear

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp(min=1e-30)).item()


def test_bert_two_layer_qat_step_matches_reference(cuda_dev):
    from transformers import BertConfig, BertModel

    g = load_golden("c4_bert2.pt")
    torch.manual_seed(3)
    model = BertModel(BertConfig(**g["cfg"]))
    for k, v in model.state_dict().items():
        if v.dtype.is_floating_point:
            assert abs(v.double().sum().item() - g["init_sum"][k]) <= 1e-9 * max(1.0, abs(g["init_sum"][k])), f"initial weights differ: {k}"
    ids = torch.randint(0, g["cfg"]["vocab_size"], (g["batch"], g["seq"]))
    G = torch.randn(g["batch"], g["seq"], g["cfg"]["hidden_size"])
    assert torch.equal(ids, g["ids"]) and torch.equal(G.bfloat16(), g["G"])
    qc = g["qcfg"]
    for name in g["qlinear_names"]:
        lin = model.get_submodule(name)
        q = QLinear(lin.in_features, lin.out_features, bias=lin.bias is not None, num_bits_feature=qc["nbits_a"], qa_mode=qc["qa_mode"],
                    num_bits_weight=qc["nbits_w"], qw_mode=qc["qw_mode"], act_clip_init_val=qc["act_clip_init_val"],
                    act_clip_init_valn=qc["act_clip_init_valn"], align_zero=g["align_zero"], device="cpu")  # fmt: skip
        with torch.no_grad():
            q.weight.copy_(lin.weight)
            q.bias.copy_(lin.bias)
        parent, _, leaf = name.rpartition(".")
        setattr(model.get_submodule(parent), leaf, q)
    model = model.to(cuda_dev)
    model.train()
    # fp32 attention through plain matmuls: the fused attention kernels take TF32 tensor-core shortcuts on fp32 inputs
    from torch.nn.attention import SDPBackend, sdpa_kernel

    with sdpa_kernel(SDPBackend.MATH):
        out = model(ids.to(cuda_dev)).last_hidden_state
        (out * G.to(cuda_dev)).sum().backward()
    torch.cuda.synchronize()
    ops.check_status(cuda_dev)

    clip_err = {}
    for name in g["qlinear_names"]:
        clip = model.get_submodule(name).quantize_weight.clip_val.detach().cpu().reshape(-1).double()
        want = g["w_clips"][name].reshape(-1).double()
        clip_err[name] = ((clip - want).abs() / want.abs()).max().item()
    worst = {"out": _rel(out.detach().cpu(), g["out"]), "w_clip": max(clip_err.values())}
    assert worst["w_clip"] < 1e-4, (worst, clip_err)
    assert worst["out"] < 3e-2, worst
    params = dict(model.named_parameters())
    # gradients that vanish in exact arithmetic (a key bias shifts every score of a row alike and drops out of the softmax)
    # are rounding noise on both sides: vectors are compared on the scale of the typical bias gradient, not on their own
    bias_norms = sorted(v.double().norm().item() for k, v in g["grads"].items() if k.endswith(".bias") and not isinstance(v, dict))
    typical = bias_norms[len(bias_norms) // 2]
    clip_pairs = []
    for n, want in g["grads"].items():
        got = params[n].grad
        assert got is not None, n
        got = got.detach().cpu()
        if isinstance(want, dict):
            r_block = _rel(got.reshape(got.shape[0], -1)[:48, :48], want["block"])
            r_norm = abs(got.double().norm().item() - want["norm"]) / max(want["norm"], 1e-30)
            worst[n] = max(r_block, r_norm)
            assert r_block < 5e-2 and r_norm < 3e-2, (n, r_block, r_norm)
        elif "clip_val" in n:
            clip_pairs.append((got.item(), want.item()))
        else:
            worst[n] = (got.double() - want.double()).norm().item() / max(want.double().norm().item(), typical)
            assert worst[n] < 5e-2, (n, worst[n])
    # The 24 clip-value gradients are each one scalar: a sum over all elements of +-g outside the clip range and of g times a
    # rounding residue inside it.  A single one moves by tens of per cent when 1 % of the activations upstream change
    # (measured: -0.44 against -0.58 for the noisiest); as a vector they must still be the reference's.
    gv, wv = torch.tensor([a for a, _ in clip_pairs]).double(), torch.tensor([b for _, b in clip_pairs]).double()
    assert len(clip_pairs) == 2 * len(g["qlinear_names"])
    worst["clip_grads_vector"] = ((gv - wv).norm() / wv.norm()).item()
    assert worst["clip_grads_vector"] < 0.3, (worst["clip_grads_vector"], clip_pairs)
    print("largest relative differences:", sorted(worst.items(), key=lambda kv: -kv[1])[:6])
