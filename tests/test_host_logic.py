"""Host-side logic that needs no GPU: deployment policy, patch state machine, gauge,
schedule choice, and the refusal to run anything on CPU tensors."""
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from lcgemm import chain_gauge, planes, qwen_policy
from lcgemm import scheme as S
from lcgemm.seams import down as down_seam


def test_qwen_stock_policy_never_imports_patch():
    for tokens in (512, 1024):
        sys.modules.pop("lcgemm.integrate.qwen_patch", None)
        assert qwen_policy.deployment_for(tokens) == "stock"
        assert qwen_policy.arm_selected_engine(tokens) is None
        assert "lcgemm.integrate.qwen_patch" not in sys.modules


def test_qwen_lc_policy_is_exact_shape():
    for tokens in (2048, 4096, 8192):
        assert qwen_policy.deployment_for(tokens) == "lc_chain"
    for tokens in (0, 513, 3072, 16384):
        with pytest.raises(ValueError):
            qwen_policy.deployment_for(tokens)
    with pytest.raises(ValueError):
        qwen_policy.install_selected_engine(object(), object(), 512)
    with pytest.raises(ValueError):
        qwen_policy.install_selected_engine(None, object(), 4096)


def test_patch_state_machine_errors():
    from lcgemm.integrate import muse_patch, qwen_patch

    for patch in (qwen_patch, muse_patch):
        if not patch._STATE["armed"]:
            with pytest.raises(RuntimeError, match="arm"):
                patch.install(object(), tokens=4096)
        if not patch._STATE["installed"]:
            with pytest.raises(RuntimeError, match="needs install"):
                patch.check_calls(1)
        assert isinstance(patch.counts(), dict)


def test_interleave_perm_matches_reference_fixture():
    f = np.load(GOLDEN / "planes.npz")
    for width in (128, 256, 640):
        assert np.array_equal(chain_gauge.interleave_perm(width).numpy(), f[f"interleave_perm.{width}"])
    with pytest.raises(ValueError):
        chain_gauge.interleave_perm(192)
    x = torch.arange(256).repeat(2, 1)
    assert torch.equal(chain_gauge.permute_k(x)[0, 64:128], torch.arange(128, 192))


def test_apply_terms_signed_sum():
    s = S.load("2x2_postsum_cse")
    frag = {(i, k): float(10 * i + k + 1) for i in range(2) for k in range(2)}
    for r in range(s.rank):
        want = sum(cf * frag[i, k] for i, k, cf in s.a_terms[r])
        assert planes.apply_terms(s.a_terms[r], frag) == want
    assert planes.apply_terms((S.Term(0, 0, -2),), frag) == -2.0


def test_rank_split_rule():
    for shape in down_seam.RANK_SPLIT_SHAPES - down_seam.HYBRID_SHAPES:
        assert down_seam.wants_rank_split(shape)
    for shape in down_seam.HYBRID_SHAPES:                          # measured exceptions
        assert not down_seam.wants_rank_split(shape)
    assert down_seam.wants_rank_split((8192, 3584, 8192))          # TP8 down: 256 tiles on 74 groups
    assert not down_seam.wants_rank_split((8192, 5120, 37888))      # 16 x 74 tiles: whole waves


def test_bare_gemm_dispatch():
    """Exact-shape dispatch of the bare rank-7 GEMM: narrow outputs form their A planes inside
    the kernel (rank-split units when whole waves would leave a short last wave), wide ones
    keep the plane pass and the postsum-CSE decomposition, odd K falls back to planes."""
    from lcgemm import _native as nat
    from lcgemm import ops

    assert ops.bare_gemm_form(4096, 5120, 17408) == ("2x2_locality_lead_single", "ahead", nat.SCHEDULE_HYBRID)
    assert ops.bare_gemm_form(8192, 5120, 17408) == ("2x2_locality_lead_single", "ahead", nat.SCHEDULE_RANK_SPLIT)
    assert ops.bare_gemm_form(2048, 6144, 16384)[1] == "ahead"
    assert ops.bare_gemm_form(4096, 34816, 5120) == ("2x2_postsum_cse", "planes", nat.SCHEDULE_HYBRID)
    assert ops.bare_gemm_form(4096, 13999, 5000) == ("2x2_postsum_cse", "planes", nat.SCHEDULE_HYBRID)
    assert ops.bare_gemm_form(4096, 5120, 17400)[1] == "planes"            # K % 128 != 0


def test_cpu_tensors_are_refused():
    s = S.load("2x2_postsum_cse")
    w = torch.zeros(64, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        planes.prepare_b(w, s)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        chain_gauge.chain_a_planes(w, s)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from lcgemm import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "absent.so")
    monkeypatch.delenv("LCGEMM_B200_AUTOBUILD", raising=False)
    with pytest.raises(RuntimeError, match="no fallback"):
        _native.lib()
