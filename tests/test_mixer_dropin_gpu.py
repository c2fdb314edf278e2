"""The four B200 backends dropped into the unmodified reference model code.

The reference's own ``SLinOSSMixer`` (slinoss/layers/mixer.py:149-223) and ``NextCharLM``
(slinoss/models/nextchar.py:265) are built from the installed reference package, once with
the reference's ``Reference*`` backends (layers/backend.py:127,186,283,407) and once, with the
same weights, with ``B200ScanBackend / B200ScanPrepBackend / B200CConv1dBackend /
B200MixerDecodeBackend``; outputs and every parameter / input gradient are compared.

Tolerances.  bf16 modules: both paths are measured against the same module evaluated in fp32
with the reference backends; a tensor passes when its relative L2 error is within the scan
contract for half inputs (2e-2) or no further from that truth than 1.5x the reference's own
bf16 run is.  fp32 modules: the reference cannot run one precision up (its scan prep mixes in
fp32 constants), so the two fp32 paths are compared with each other: output <= 1e-4, gradients
<= 2e-3.  The spread comes from the reference's fp32 tap formulas ((rho - 1)/z cancels for
small |z|); tests/test_prep_conv_gpu.py measures the kernels against a float64 oracle of the
same maps, which is the tighter statement.
"""

from __future__ import annotations

import copy

import pytest
import torch

from ref_util import import_reference, use_b200_backends, use_reference_backends

pytestmark = pytest.mark.gpu


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double(), b.detach().double()
    den = b.norm().item()
    return (a - b).norm().item() / den if den > 0 else (a - b).norm().item()


def _run_layer(mixer, x, w):
    x = x.detach().clone().requires_grad_(True)
    for p in mixer.parameters():
        p.grad = None
    y = mixer(x)
    (y.float() * w.float()).sum().backward()
    grads = {"x": x.grad.detach().clone()}
    grads.update({n: p.grad.detach().clone() for n, p in mixer.named_parameters() if p.grad is not None})
    return y.detach(), grads


def _make_mixers(dtype, *, d_model, d_state, expand, chunk, seed):
    import_reference()
    from slinoss.layers import SLinOSSMixer

    torch.manual_seed(seed)
    ref = SLinOSSMixer(d_model, d_state=d_state, expand=expand, d_head=64, d_conv=4, chunk_size=chunk,
                       device="cuda", dtype=dtype).train()
    use_reference_backends(ref)
    ours = copy.deepcopy(ref)
    assert use_b200_backends(ours) == 1
    return ref, ours


def test_mixer_layer_bf16_matches_reference_backends():
    """Reduced form of the single-layer configuration (d_model 768, 12 heads of 64, d_state 64,
    conv width 4, chunk 64, bf16 with fp32 scan state; batch 2, 512 tokens)."""
    ref, ours = _make_mixers(torch.bfloat16, d_model=768, d_state=64, expand=1, chunk=64, seed=0)
    assert ref.n_heads == 12
    truth = copy.deepcopy(ref).float()
    use_reference_backends(truth)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((2, 512, 768), device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn((2, 512, 768), device="cuda", generator=g)
    y_t, g_t = _run_layer(truth, x.float(), w)
    y_r, g_r = _run_layer(ref, x, w)
    y_o, g_o = _run_layer(ours, x, w)
    assert set(g_o) == set(g_r) == set(g_t)
    report = {"y": (_rel(y_o, y_t), _rel(y_r, y_t))}
    for name in g_t:
        report[name] = (_rel(g_o[name], g_t[name]), _rel(g_r[name], g_t[name]))
    for name, (eo, er) in report.items():
        print(f"[mixer bf16] {name:32s} b200 vs fp32 truth {eo:.3e}   reference bf16 vs truth {er:.3e}")
    bad = {n: v for n, v in report.items() if not (v[0] <= 2e-2 or v[0] <= 1.5 * v[1])}
    assert not bad, bad


def test_mixer_layer_fp32_matches_reference_backends():
    """fp32 module, ragged length (not a multiple of the chunk), expand 2."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref, ours = _make_mixers(torch.float32, d_model=128, d_state=16, expand=2, chunk=32, seed=3)
        g = torch.Generator(device="cuda").manual_seed(4)
        x = torch.randn((2, 77, 128), device="cuda", generator=g)
        w = torch.randn((2, 77, 128), device="cuda", generator=g)
        y_r, g_r = _run_layer(ref, x, w)
        y_o, g_o = _run_layer(ours, x, w)
        errs = {"y": _rel(y_o, y_r)}
        errs.update({n: _rel(g_o[n], g_r[n]) for n in g_r})
        for n, e in errs.items():
            print(f"[mixer fp32] {n:32s} {e:.3e}")
        assert errs["y"] <= 1e-4, errs
        assert max(errs.values()) <= 2e-3, errs
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_mixer_streaming_segments_match_single_pass():
    """Two segments chained through ``SLinOSSMixerState`` (conv state + scan state) equal one
    pass over the whole sequence (pattern of tests/test_mixer.py:411-461 of the reference)."""
    _, ours = _make_mixers(torch.float32, d_model=128, d_state=64, expand=2, chunk=32, seed=5)
    ours.eval()
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn((2, 49, 128), device="cuda", generator=g)
    with torch.no_grad():
        y_full, st_full = ours(x, return_state=True)
        y_a, st = ours(x[:, :17, :], return_state=True)
        y_b, st = ours(x[:, 17:, :], state=st, return_state=True)
    y_seg = torch.cat([y_a, y_b], dim=1)
    assert _rel(y_seg, y_full) <= 1e-5
    assert _rel(st.scan.state, st_full.scan.state) <= 1e-5
    assert torch.equal(st.scan.b_prev, st_full.scan.b_prev)
    assert torch.equal(st.scan.u_prev, st_full.scan.u_prev)
    assert torch.equal(st.conv, st_full.conv)


def test_nextchar_lm_step_matches_reference_backends():
    """Reduced form of the language-model configuration (the reference's ``NextCharLM``, byte
    vocabulary, uniform random tokens): 2 layers, d_model 256, 4 heads, d_state 128, bf16;
    one forward + cross-entropy + backward with every mixer on the B200 backends against the
    same model on the reference backends."""
    import_reference()
    from slinoss.models.nextchar import NextCharLM

    torch.manual_seed(7)
    kw = dict(vocab_size=256, block_size=256, d_model=256, n_layers=2, d_state=128, expand=1, d_head=64,
              d_conv=4, chunk_size=64)
    ref = NextCharLM(**kw).to(device="cuda", dtype=torch.bfloat16)
    use_reference_backends(ref)
    ours = copy.deepcopy(ref)
    assert use_b200_backends(ours) == 2
    truth = copy.deepcopy(ref).float()
    use_reference_backends(truth)
    g = torch.Generator(device="cuda").manual_seed(8)
    xb = torch.randint(0, 256, (4, 256), device="cuda", generator=g)
    yb = torch.randint(0, 256, (4, 256), device="cuda", generator=g)

    def step(model):
        model.zero_grad(set_to_none=True)
        logits = model(xb)
        loss = torch.nn.functional.cross_entropy(logits.float().view(-1, 256), yb.view(-1))
        loss.backward()
        return loss.detach(), {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}

    l_t, g_t = step(truth)
    l_r, g_r = step(ref)
    l_o, g_o = step(ours)
    print(f"[nextchar] loss truth {l_t.item():.5f} reference bf16 {l_r.item():.5f} b200 {l_o.item():.5f}")
    assert abs(l_o.item() - l_t.item()) <= max(2e-2 * abs(l_t.item()), 1.5 * abs(l_r.item() - l_t.item()))
    assert set(g_o) == set(g_r)
    # whole-model gradient: norm of the concatenated error against the fp32 truth
    num_o = sum((g_o[n].double() - g_t[n].double()).square().sum().item() for n in g_t) ** 0.5
    num_r = sum((g_r[n].double() - g_t[n].double()).square().sum().item() for n in g_t) ** 0.5
    den = sum(g_t[n].double().square().sum().item() for n in g_t) ** 0.5
    print(f"[nextchar] gradient error vs fp32 truth: b200 {num_o / den:.3e}, reference bf16 {num_r / den:.3e}")
    assert num_o / den <= max(2e-2, 1.5 * num_r / den)
    for n in g_o:
        assert torch.isfinite(g_o[n]).all(), n
