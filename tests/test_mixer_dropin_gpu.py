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

import contextlib
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


@contextlib.contextmanager
def _reference_taps_in_double():
    """Inside this context the installed reference evaluates its first-order-hold taps in
    float64 (same closed form, ``kappa1 = (e^z - 1)/z``, ``kappa2 = (e^z (z-1) + 1)/z^2``, results
    cast back to fp32).  The reference's own fp32 evaluation of ``kappa2`` cancels to a relative
    error of about eps/|z|^2 (and its autograd derivative to eps/|z|^3) for the small ``|z|`` a
    default-initialised layer produces, so an fp32 reference run is not a usable truth for the
    gradients of the scan-prep parameters; this gives one."""
    import slinoss.layers.scanprep as layer_mod
    import slinoss.ops.scanprep.reference as ref_mod

    def taps64(dt_f, log_r_f, theta_f, rho, *, eps):
        z = torch.complex(log_r_f.double(), theta_f.double())
        e = torch.exp(z)
        tiny = (z.real.square() + z.imag.square()) < 1e-8
        zs = torch.where(tiny, torch.ones_like(z), z)
        k1 = torch.where(tiny, 1 + z / 2 + z * z / 6, (e - 1) / zs)
        k2 = torch.where(tiny, 0.5 + z / 3 + z * z / 8, (e * (zs - 1) + 1) / (zs * zs))
        k_prev = dt_f.double() * k2
        k_curr = dt_f.double() * k1 - k_prev
        return ref_mod._pack_complex(k_prev), ref_mod._pack_complex(k_curr)

    saved = (layer_mod._foh_taps_from_normalized, ref_mod._foh_taps_from_normalized)
    layer_mod._foh_taps_from_normalized = ref_mod._foh_taps_from_normalized = taps64
    try:
        yield
    finally:
        layer_mod._foh_taps_from_normalized, ref_mod._foh_taps_from_normalized = saved


def test_mixer_layer_fp32_matches_reference_backends():
    """fp32 module, ragged length (not a multiple of the chunk), expand 2.  Three-way: the B200
    backends and the reference's fp32 backends against the reference with its taps in double.
    The layer output must agree with both to 1e-4 and every gradient must be within 2e-5 of the
    truth (measured ~1e-6, where the reference's own fp32 run is up to 2.4e-3 away from it)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref, ours = _make_mixers(torch.float32, d_model=128, d_state=16, expand=2, chunk=32, seed=3)
        truth = copy.deepcopy(ref)
        use_reference_backends(truth)
        g = torch.Generator(device="cuda").manual_seed(4)
        x = torch.randn((2, 77, 128), device="cuda", generator=g)
        w = torch.randn((2, 77, 128), device="cuda", generator=g)
        with _reference_taps_in_double():
            y_t, g_t = _run_layer(truth, x, w)
        y_r, g_r = _run_layer(ref, x, w)
        y_o, g_o = _run_layer(ours, x, w)
        report = {"y": (_rel(y_o, y_t), _rel(y_r, y_t), _rel(y_o, y_r))}
        for n in g_t:
            report[n] = (_rel(g_o[n], g_t[n]), _rel(g_r[n], g_t[n]), _rel(g_o[n], g_r[n]))
        for n, (eo, er, eor) in report.items():
            print(f"[mixer fp32] {n:32s} b200 vs truth {eo:.3e}   reference fp32 vs truth {er:.3e}   "
                  f"b200 vs reference fp32 {eor:.3e}")
        assert report["y"][0] <= 1e-4 and report["y"][2] <= 1e-4, report["y"]
        bad = {n: v for n, v in report.items() if not v[0] <= 2e-5}
        assert not bad, bad
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


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_mixer_step_matches_full_forward(dtype, tol):
    """Token-by-token ``mixer.step`` (conv step through ``slx_cconv1d_update``, scan step through
    ``B200MixerDecodeBackend``) against one ``forward`` over the same tokens with the same backends
    (pattern of the reference's tests/test_mixer.py:543-576)."""
    _, ours = _make_mixers(dtype, d_model=128, d_state=64, expand=2, chunk=32, seed=9)
    ours.eval()
    g = torch.Generator(device="cuda").manual_seed(10)
    x = torch.randn((3, 11, 128), device="cuda", generator=g).to(dtype)
    with torch.no_grad():
        y_full, st_full = ours(x, return_state=True)
        st = ours.init_state(x.shape[0], device=x.device, dtype=x.dtype)
        pieces = []
        for t in range(x.shape[1]):
            y_t, st = ours.step(x[:, t, :], st)
            pieces.append(y_t.unsqueeze(1))
    y_step = torch.cat(pieces, dim=1)
    errs = dict(y=_rel(y_step, y_full), conv=_rel(st.conv, st_full.conv),
                state=_rel(st.scan.state, st_full.scan.state), b_prev=_rel(st.scan.b_prev, st_full.scan.b_prev),
                u_prev=_rel(st.scan.u_prev, st_full.scan.u_prev))
    print("[mixer step]", dtype, {k: f"{v:.2e}" for k, v in errs.items()})
    assert max(errs.values()) <= tol, errs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
def test_conv_update_matches_reference_conv_step(dtype, width):
    """``cconv1d_update_b200`` against the reference's own conv step arithmetic
    (``_apply_cconv_reference`` on a one-token sequence + SiLU, mixer.py:660-676), three tokens in
    a row with the rolling state, out of place and in place."""
    import_reference()
    from slinoss.layers import SLinOSSMixer
    from slinoss.layers.backend import ReferenceCConv1dBackend

    import slinoss_b200 as sb

    torch.manual_seed(width)
    mixer = SLinOSSMixer(96, d_state=16, expand=2, d_head=64, d_conv=width, device="cuda", dtype=dtype,
                         cconv_backend=ReferenceCConv1dBackend())
    b, C = 5, mixer.d_inner
    st_ref = torch.randn((b, C, width - 1), device="cuda").to(dtype)
    st_out, st_in = st_ref.clone(), st_ref.clone().contiguous()
    wide = torch.randn((3, b, 2 * C + 7), device="cuda").to(dtype)   # x is a column slice of a wider row
    for t in range(3):
        x = wide[t, :, 3:3 + C]
        with torch.no_grad():
            y_seq, st_ref = mixer._apply_cconv_reference(x.unsqueeze(1), st_ref)
            y_ref = torch.nn.functional.silu(y_seq[:, 0, :])
        y1, st_out = sb.cconv1d_update_b200(x, mixer.dw_weight, mixer.dw_bias, st_out, activation="silu")
        y2, st_in2 = sb.cconv1d_update_b200(x, mixer.dw_weight, mixer.dw_bias, st_in, activation="silu", inplace=True)
        assert st_in2 is st_in
        tol = 1e-6 if dtype == torch.float32 else 1e-2
        assert _rel(y1, y_ref) <= tol and _rel(y2, y_ref) <= tol
        assert torch.equal(st_out, st_ref) and torch.equal(st_in, st_ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_skip_matches_reference_glue(dtype):
    """``gate_skip_b200`` (skip, re-layout, SiLU gate in one pass; gate read as a column slice of a wider
    projection row) against ``SLinOSSMixer._apply_gate_skip`` (mixer.py:585-599), forward and all four
    gradients."""
    import_reference()
    from slinoss.layers import SLinOSSMixer

    import slinoss_b200 as sb

    torch.manual_seed(11)
    mixer = SLinOSSMixer(192, d_state=16, expand=2, d_head=64, device="cuda", dtype=dtype)
    with torch.no_grad():
        mixer.skip.copy_(torch.randn_like(mixer.skip))
    b, T, H, P = 2, 75, mixer.n_heads, mixer.d_head
    g = torch.Generator(device="cuda").manual_seed(12)
    wide = torch.randn((b, T, 2 * H * P + 8), device="cuda", generator=g).to(dtype)
    leaves_r = [torch.randn((b, H, T, P), device="cuda", generator=g).to(dtype).requires_grad_(True) for _ in range(2)]
    gate_r = wide[..., 8:8 + H * P].detach().clone().requires_grad_(True)
    w = torch.randn((b, T, H * P), device="cuda", generator=g).to(dtype)
    out_r = mixer._apply_gate_skip(leaves_r[0], leaves_r[1], gate_r, b, T)
    gr = torch.autograd.grad(out_r, leaves_r + [gate_r, mixer.skip], w)
    leaves_o = [t.detach().clone().requires_grad_(True) for t in leaves_r]
    wide_o = wide.detach().clone().requires_grad_(True)
    skip_o = mixer.skip.detach().clone().requires_grad_(True)
    out_o = sb.gate_skip_b200(leaves_o[0], leaves_o[1], wide_o[..., 8:8 + H * P], skip_o)
    go = torch.autograd.grad(out_o, leaves_o + [wide_o, skip_o], w)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    errs = dict(out=_rel(out_o, out_r), dy=_rel(go[0], gr[0]), du=_rel(go[1], gr[1]),
                dgate=_rel(go[2][..., 8:8 + H * P], gr[2]), dskip=_rel(go[3], gr[3]))
    print("[gate_skip]", dtype, {k: f"{v:.2e}" for k, v in errs.items()})
    assert max(errs.values()) <= tol, errs
    assert float(go[2][..., :8].abs().max()) == 0.0   # nothing leaks outside the gate's columns


def test_mixer_fused_glue_matches_unfused():
    """``use_b200_backends(..., fuse_glue=True)``: SiLU inside the conv kernel and the one-pass gate/skip.
    The fused layer skips two roundings to bf16 that the reference's forward makes, so the two bf16
    layers are compared three-way against the fp32 reference layer: every tensor of the fused layer
    must be within 2e-2 of the truth or no further from it than 1.5x the unfused layer.  The per-head
    bias gradients of the scan prep (4 numbers each here, every one a sum of ~1e5 signed terms that
    nearly cancel) move by a few percent between any two bf16 evaluations of the layer; they get 5e-2."""
    import slinoss_b200 as sb

    ref, plain = _make_mixers(torch.bfloat16, d_model=256, d_state=64, expand=1, chunk=64, seed=13)
    fused = copy.deepcopy(plain)
    assert sb.use_b200_backends(fused, fuse_glue=True) == 1
    truth = copy.deepcopy(ref).float()
    use_reference_backends(truth)
    g = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn((2, 300, 256), device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn((2, 300, 256), device="cuda", generator=g)
    y_t, g_t = _run_layer(truth, x.float(), w)
    y_p, g_p = _run_layer(plain, x, w)
    y_f, g_f = _run_layer(fused, x, w)
    assert set(g_f) == set(g_p) == set(g_t)
    report = {"y": (_rel(y_f, y_t), _rel(y_p, y_t))}
    for n in g_t:
        report[n] = (_rel(g_f[n], g_t[n]), _rel(g_p[n], g_t[n]))
    for n, (ef, ep) in report.items():
        print(f"[fused glue] {n:32s} fused vs fp32 truth {ef:.3e}   unfused vs truth {ep:.3e}")
    small = {n for n in g_t if g_t[n].numel() <= 16}
    bad = {n: v for n, v in report.items()
           if not (v[0] <= 2e-2 or v[0] <= 1.5 * v[1] or (n in small and v[0] <= 5e-2))}
    assert not bad, bad
    # streaming state is carried the same way
    with torch.no_grad():
        y_a, st = fused(x[:, :100], return_state=True)
        y_b, st = fused(x[:, 100:], state=st, return_state=True)
        y_full, st_full = plain(x, return_state=True)
    assert _rel(torch.cat([y_a, y_b], dim=1), y_full) <= 1e-2
    assert _rel(st.scan.state, st_full.scan.state) <= 1e-2 and torch.equal(st.conv, st_full.conv)


def test_aligned_projection_gives_the_same_rows_on_16_byte_boundaries():
    """``use_b200_backends`` runs an input projection whose width is not a multiple of 8 (4764 at
    d_model 768, 12 heads, d_state 64) on a zero-padded weight: same values as the plain ``nn.Linear``
    (up to the rounding of a different GEMM kernel), rows 4768 apart, parameters untouched, gradients
    of weight and input as before."""
    ref, ours = _make_mixers(torch.bfloat16, d_model=768, d_state=64, expand=1, chunk=64, seed=21)
    assert int(ours.in_proj.out_features) == 4764 and "forward" in vars(ours.in_proj) and "forward" not in vars(ref.in_proj)
    g = torch.Generator(device="cuda").manual_seed(22)
    x = torch.randn((2, 96, 768), device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
    w = torch.randn((2, 96, 4764), device="cuda", generator=g).to(torch.bfloat16)
    y_r = ref.in_proj(x)
    y_o = ours.in_proj(x)
    assert tuple(y_o.shape) == (2, 96, 4764) and y_o.stride(1) == 4768 and y_r.stride(1) == 4764
    assert _rel(y_o, y_r) <= 4e-3
    gx_r, gw_r = torch.autograd.grad(y_r, [x, ref.in_proj.weight], w)
    gx_o, gw_o = torch.autograd.grad(y_o, [x, ours.in_proj.weight], w)
    assert gw_o.shape == gw_r.shape == (4764, 768)
    assert _rel(gx_o, gx_r) <= 4e-3 and _rel(gw_o, gw_r) <= 4e-3
    # a projection that is already aligned keeps the stock forward
    _, other = _make_mixers(torch.bfloat16, d_model=512, d_state=64, expand=1, chunk=64, seed=23)   # width 3176
    assert int(other.in_proj.out_features) % 8 == 0 and "forward" not in vars(other.in_proj)
