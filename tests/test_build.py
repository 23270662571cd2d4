"""Which files a kernel library is built from, and that an edit to any of them changes the library's name.  No GPU needed."""
from pathlib import Path

from cisr_b200.ops import build


def names(source):
    return [p.name for p in build.source_closure(build.CSRC / source)]


def test_the_include_closure_follows_every_kind_of_included_file():
    # a .cu file that includes another .cu file and a .h beside the .cuh headers
    assert names("attention_static_scratch.cu") == ["attention.cu", "attention_static_scratch.cu", "attention_static_scratch.h",
                                                    "common.cuh"]
    # headers included by headers
    assert {"tcgen05.cuh", "tma.cuh", "common.cuh"} <= set(names("gemm_tcgen05.cu"))
    assert names("elementwise.cu") == ["common.cuh", "elementwise.cu"]


def test_an_edit_to_an_included_file_renames_the_library(tmp_path, monkeypatch):
    (tmp_path / "top.cu").write_text('#include "mid.cu"\n#include "limit.h"\nint top;\n')
    (tmp_path / "mid.cu").write_text('  #  include "deep.cuh"\nint mid;\n')
    (tmp_path / "deep.cuh").write_text("int deep;\n")
    (tmp_path / "limit.h").write_text("#define LIMIT 8\n")
    (tmp_path / "other.cu").write_text("int other;\n")
    monkeypatch.setattr(build, "CSRC", tmp_path)
    monkeypatch.setattr(build, "_build_dir", tmp_path)
    first = build.library_path("top.cu", {"D": 1})
    assert first == build.library_path("top.cu", {"D": 1})
    assert first != build.library_path("top.cu", {"D": 2})
    (tmp_path / "other.cu").write_text("int other = 1;\n")               # not included: the name stays
    assert build.library_path("top.cu", {"D": 1}) == first
    for edited, text in (("limit.h", "#define LIMIT 16\n"), ("deep.cuh", "int deeper;\n"), ("mid.cu", '#include "deep.cuh"\nint mid2;\n')):
        before = build.library_path("top.cu", {"D": 1})
        (tmp_path / edited).write_text(text)
        assert build.library_path("top.cu", {"D": 1}) != before, edited


def test_a_new_build_removes_the_superseded_ones_of_the_same_kernel_only(tmp_path):
    keep = ["libcisr_gemm_0123456789abcdef.so", "libcisr_gemm_cisr_trace1_0123456789abcdef.so", "libcisr_gemm_wide_0123456789abcdef.so",
            "libcisr_attention_head_dim128_0123456789abcdef.so"]
    drop = ["libcisr_gemm_fedcba9876543210.so", "libcisr_gemm_00000000aaaaaaaa.so"]
    for name in keep + drop + ["libcisr_attention_head_dim16_0123456789abcdef.so", "libcisr_attention_head_dim16_ffffffffffffffff.so"]:
        (tmp_path / name).write_bytes(b"")
    build._drop_superseded(tmp_path / "libcisr_gemm_0123456789abcdef.so")
    build._drop_superseded(tmp_path / "libcisr_attention_head_dim16_ffffffffffffffff.so")
    assert sorted(p.name for p in tmp_path.iterdir()) == sorted(keep + ["libcisr_attention_head_dim16_ffffffffffffffff.so"])
