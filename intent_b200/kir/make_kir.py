"""Regenerates the kernel IR (KIR) texts in this directory with the reference frontend.

Run where the reference checkout is importable:

    PYTHONPATH=<reference>/python python intent_b200/kir/make_kir.py

The frontend (python/intent/frontend/compilation/compiler.py:88-100) is pure
Python; its output is the text the native compile step receives on stdin
(python/intent/compiler/toolchain.py:212-219).  Source locations are rewritten
to be relative to the reference checkout so the fixtures do not depend on
where it is mounted.

``csr_spmm`` has static module-level extents in the reference
(python/intent/examples/kernels/sparse/csr_spmm.py:5-9: 8192 rows).  The
262144-row instance is produced by executing the reference's own module source
with those five constants changed; nothing of the kernel body is restated here.
"""
from pathlib import Path
import re
import sys

import intent
from intent.examples.kernels.contraction import gemm as gemm_kernels
from intent.examples.kernels.normalization import layer_norm, softmax
from intent.examples.kernels.backward import attention as attention_backward_kernels
from intent.examples.kernels.backward import layer_norm as layer_norm_backward_kernels
from intent.examples.kernels.backward import softmax as softmax_backward_kernels
from intent.examples.kernels.sparse import csr_spmm, csr_spmv
from intent.examples.kernels.streaming import attention

CASES = {
    "stable_softmax": (softmax.stable_softmax, None),
    "stable_softmax_f16": (softmax.stable_softmax_f16, None),
    "chunked_softmax_bf16": (softmax.chunked_softmax_bf16, None),
    "layer_norm_f16": (layer_norm.layer_norm_f16, None),
    "layer_norm_bf16": (layer_norm.layer_norm_bf16, None),
    "weighted_layer_norm": (layer_norm.weighted_layer_norm, None),
    "gemm": (gemm_kernels.gemm, {"ACTIVATION": gemm_kernels.Activation.NONE}),
    "gemm_relu": (gemm_kernels.gemm, {"ACTIVATION": gemm_kernels.Activation.RELU}),
    "bf16_gemm": (gemm_kernels.bf16_gemm, None),
    "flash_attention_bf16_fwd": (attention.flash_attention_bf16_fwd, {"HEAD_GROUP": 1, "CAUSAL": True}),
    "flash_attention_fwd": (attention.flash_attention_fwd, {"CAUSAL": True}),
    "flash_attention_fwd_noncausal": (attention.flash_attention_fwd, {"CAUSAL": False}),
    "flash_gqa_attention_fwd": (attention.flash_gqa_attention_fwd, {"HEAD_GROUP": 4, "CAUSAL": True}),
    "csr_spmm": (csr_spmm.csr_spmm, None),
    "csr_spmv": (csr_spmv.csr_spmv, None),
    "softmax_backward": (softmax_backward_kernels.softmax_backward, None),
    "layer_norm_backward_rows": (layer_norm_backward_kernels.layer_norm_backward_rows, None),
    "layer_norm_backward_reduce": (layer_norm_backward_kernels.layer_norm_backward_reduce, None),
    "attention_backward_delta": (attention_backward_kernels.attention_backward_delta, None),
    "attention_backward_dkdv": (attention_backward_kernels.attention_backward_dkdv, {"HEAD_GROUP": 4, "CAUSAL": True}),
    "attention_backward_dkdv_noncausal": (attention_backward_kernels.attention_backward_dkdv,
                                          {"HEAD_GROUP": 1, "CAUSAL": False}),
    "attention_backward_dq": (attention_backward_kernels.attention_backward_dq, {"HEAD_GROUP": 4, "CAUSAL": True}),
    "attention_backward_dq_noncausal": (attention_backward_kernels.attention_backward_dq,
                                        {"HEAD_GROUP": 1, "CAUSAL": False}),
    # kernels outside the five families: the compile step must refuse them
    "gemm_f32": (gemm_kernels.gemm_f32, None),
}


def resized_csr_spmm(rows: int, columns: int, per_row: int, features: int):
    import importlib.util
    import tempfile

    source = Path(csr_spmm.__file__).read_text(encoding="utf-8")
    for name, value in (("ROWS", rows), ("COLUMNS", columns), ("NONZEROS_PER_ROW", per_row),
                        ("FEATURES", features)):
        source, count = re.subn(rf"^{name} = \d+$", f"{name} = {value}", source, flags=re.M)
        assert count == 1, name
    directory = Path(tempfile.mkdtemp())
    path = directory / "csr_spmm_resized.py"
    path.write_text(source, encoding="utf-8")
    spec = importlib.util.spec_from_file_location("csr_spmm_resized", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.csr_spmm, str(path), "python/intent/examples/kernels/sparse/csr_spmm.py"


def main() -> None:
    out = Path(__file__).resolve().parent
    root = str(Path(intent.__file__).resolve().parents[2])
    for name, (definition, constexprs) in CASES.items():
        text = intent.lower_to_mlir(definition, constexprs=constexprs)
        text = text.replace(root + "/", "")
        (out / f"{name}.mlir").write_text(text, encoding="utf-8")
        print(name, len(text))
    definition, temporary, original = resized_csr_spmm(262144, 262144, 32, 128)
    text = intent.lower_to_mlir(definition).replace(temporary, original)
    (out / "csr_spmm_262144.mlir").write_text(text, encoding="utf-8")
    print("csr_spmm_262144", len(text))


if __name__ == "__main__":
    main()
