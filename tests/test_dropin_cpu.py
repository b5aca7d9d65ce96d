"""The drop-in itself: ``come_b200.cuda_extension.install()`` registered under the reference's import names, inside an
unmodified checkout of the reference, must make the reference's own lookup of its accelerated entry points
(``src/utility/feature.py:104-168``) land on this library's stand-ins.

The checkout is taken from the environment variable ``COME_REFERENCE_ROOT``; without it the tests are skipped.  They run
in a child process (the reference's ``src`` package and the stubs of its uninstalled dependencies stay out of this one).
"""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("COME_REFERENCE_ROOT", "")

pytestmark = pytest.mark.skipif(not (REF and os.path.isdir(os.path.join(REF, "src", "accelerate"))),
                                reason="COME_REFERENCE_ROOT does not point at a checkout of the reference")

PRELUDE = textwrap.dedent("""
    import sys, types
    def stub(name, **attrs):
        m = types.ModuleType(name); m.__dict__.update(attrs); sys.modules[name] = m; return m
    stub("hydra"); sys.modules["hydra"].utils = stub("hydra.utils", instantiate=lambda *a, **k: None)
    stub("omegaconf", DictConfig=dict, OmegaConf=object); stub("pypose")
    sys.path.insert(0, {root!r}); sys.path.insert(0, {ref!r})
    import come_b200.cuda_extension as ce
    ce.install()
""")


def _run(body: str) -> str:
    code = PRELUDE.format(root=ROOT, ref=REF) + textwrap.dedent(body)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_reference_lookup_lands_on_the_stand_ins():
    out = _run("""
        from src.utility.feature import CUDAExtension
        assert CUDAExtension.is_available()
        import src.cuda_extension as rce
        from come_b200 import co_me_cuext, flash_attn
        assert rce is ce and rce.co_me_cuext is co_me_cuext
        # the reference's merger module attaches its two Python wrappers to the extension module and its decorator
        # resolves them from there (co_me.py:131-149,225-238; feature.py:160-168)
        from src.accelerate.token_merger import co_me
        assert co_me.co_me_cuext is co_me_cuext
        assert co_me_cuext.co_me_token_merge_cuda_entrypoint is co_me.co_me_token_merge_cuda_entrypoint
        assert co_me_cuext.token_split_py_wrapper is co_me._token_split_cuda
        assert co_me.func_token_merge.__wrapped__ is not co_me.func_token_merge  # dispatching wrapper, not the fallback
        # the attention modules import three names from the package (bias_attention.py:15-16, plain_attention.py:6-7)
        from src.accelerate.vggt.module import bias_attention, plain_attention
        assert bias_attention.flash_attn_varlen_qkvpacked_func_w_perkey_bias is flash_attn.flash_attn_varlen_qkvpacked_func_w_perkey_bias
        assert plain_attention.flash_attn_varlen_qkvpacked_func is flash_attn.flash_attn_varlen_qkvpacked_func
        assert bias_attention.infer_flash_attn_varlen_max_seqlen is flash_attn.infer_flash_attn_varlen_max_seqlen
        print("resolved")
    """)
    assert "resolved" in out


def test_reference_fallback_still_runs_under_disable():
    """With the stand-ins installed, ``CUDAExtension.disable()`` still selects the reference's PyTorch fallback (what the
    golden fixtures are generated with), and a CPU tensor handed to the accelerated path is refused, not silently
    computed somewhere else."""
    out = _run("""
        import torch
        from src.utility.feature import CUDAExtension
        from src.accelerate.token_merger.co_me import func_token_merge
        tokens = torch.arange(2 * 7 * 2, dtype=torch.float32).reshape(2, 7, 2)
        mask = torch.tensor([[True, False], [False, True]])
        with CUDAExtension.disable():
            jag, rev = func_token_merge(tokens, 1, 3, mask)
        assert jag.tokens.shape[1] == 2 * 7 - 2 * 2 and rev.shape[0] == 14
        try:
            func_token_merge(tokens, 1, 3, mask)
        except RuntimeError as e:
            assert "CUDA" in str(e) or "cuda" in str(e), e
            print("refused")
    """)
    assert "refused" in out
