"""The binding INTEGRATION.md shows a maintainer of the reference is executed as written: the code block is cut
out of the document, pointed at the built library and bound onto an UNMODIFIED upstream module (the copy the recipe
oracle/build_ref.py installs under oracle/_ref) holding an upstream state on the GPU.  Its result must agree with
upstream's own ``attend_step`` (PyTorch path) within the bf16 tolerance."""
import os
import re
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _example_source() -> str:
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    src = [b for b in blocks if "def fused_attend_step" in b]
    assert len(src) == 1, "INTEGRATION.md should hold exactly one code block defining fused_attend_step"
    return src[0]


def test_integration_document_holds_the_binding_example():
    src = _example_source()
    assert "coda_b200_decode_attend" in src and "class LayerCfg" in src and "class StatePtrs" in src
    compile(src, "INTEGRATION.md", "exec")                       # valid Python as printed


@pytest.mark.gpu
@pytest.mark.parametrize("kw", [
    dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=48, num_landmarks_exact=16, num_landmarks_summary=16),
    dict(embed_dim=1024, num_heads=8, num_kv_heads=4, window=64, num_landmarks_exact=16, num_landmarks_summary=16,
         rope_interleaved=False, head_norm_mode="identity", rope_base=1e6),
])
def test_binding_example_on_the_upstream_module_matches_upstream_attend_step(kw):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_ref
    if not build_ref.available():
        pytest.skip("oracle/_ref (the installed upstream package) is not present")
    Upstream = build_ref.load()
    sys.path.insert(0, os.path.join(ROOT, "coda-gqa-l_b200"))
    from coda_gqa_l_b200 import _lib
    src = _example_source().replace('C.CDLL("libcoda_b200.so")', f'C.CDLL({_lib.LIB_PATH!r})')
    ns = {}
    exec(compile(src, "INTEGRATION.md", "exec"), ns)
    fused_attend_step = ns["fused_attend_step"]

    torch.manual_seed(0)
    m = Upstream(**kw).eval()
    with torch.no_grad():
        for p_ in m.parameters():                                 # non-trivial theta / lambda / norm weights
            p_.add_(torch.randn_like(p_) * 0.05)
    m = m.to(torch.bfloat16).cuda()
    B = 3
    x = (torch.randn(B, 200, kw["embed_dim"], device="cuda") * 0.5).to(torch.bfloat16)
    with torch.no_grad():
        st = m.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
        _, st = m.prefill_chunked(x[:, :160], st, block_size=32)                  # upstream's own prefill on the GPU
        for t in range(160, 170):
            xt = x[:, t:t + 1]
            y_ref = m.attend_step(xt, st)                                         # upstream, PyTorch path
            q_raw = m.q_proj(xt).reshape(B, -1).contiguous()
            lam_logit = m.lambda_proj(xt).reshape(B, -1).contiguous()
            heads = fused_attend_step(m, q_raw, lam_logit, st, st.pos)            # the document's binding
            y = m.o_proj(heads).view(B, 1, -1)
            err = (y.double() - y_ref.double()).norm() / y_ref.double().norm()
            assert float(err) < 2e-2, f"token {t}: rel err {float(err):.3e}"
            _, st = m.step(xt, st)                                                # upstream advances its own state
