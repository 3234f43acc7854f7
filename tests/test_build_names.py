"""How kernel libraries are named and found, without compiling anything: one library per source and set of
macros, the name carries a hash of source, headers and flags (so an edited kernel is never served from an old
build), every source of csrc/ is known to the builder, and the flags ask for sm_100a and nothing else."""
import os

import pytest

from mlx_lm_b200.ops import build


def test_names_of_plain_libraries_and_variants():
    assert build._split("attention") == ("attention", [])
    assert build._split("attention:MLXB_X=8,OTHER=1") == ("attention", ["MLXB_X=8", "OTHER=1"])
    plain, variant = build.lib_path("attention"), build.lib_path("attention:MLXB_X=8")
    other = build.lib_path("attention:MLXB_X=4")
    assert len({plain, variant, other}) == 3
    assert os.path.basename(variant).startswith("attention.MLXB_X_8-") and variant.endswith(".so")
    assert os.path.dirname(plain) == build.build_dir()
    assert build.lib_path("attention") == build.lib_path("attention")        # a pure function of the sources


def test_hash_follows_the_source(tmp_path, monkeypatch):
    before = build._digest("embed")
    src = os.path.join(build.CSRC, "embed.cu")
    with open(src) as f:
        text = f.read()
    fake = tmp_path / "csrc"
    fake.mkdir()
    for name in os.listdir(build.CSRC):
        if name.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(build.CSRC, name)) as f, open(fake / name, "w") as g:
                g.write(f.read())
    monkeypatch.setattr(build, "CSRC", str(fake))
    assert build._digest("embed") == before                      # same bytes, same hash, wherever they lie
    with open(fake / "embed.cu", "w") as f:
        f.write(text + "\n// edited\n")
    assert build._digest("embed") != before
    with open(fake / "embed.cu", "w") as f:
        f.write(text)
    with open(fake / "common.cuh", "a") as f:
        f.write("\n// edited header\n")
    assert build._digest("embed") != before                      # headers count too


def test_every_source_is_known_and_flags_are_for_sm_100a():
    sources = set(build.all_sources())
    on_disk = {f[:-3] for f in os.listdir(build.CSRC) if f.endswith(".cu")}
    assert sources == on_disk and {"attention", "gemm_tcgen05", "gemm_smallm", "norm", "embed", "sampling"} <= sources
    flags = " ".join(build.NVCC_FLAGS)
    assert "arch=compute_100a,code=sm_100a" in flags and "-lineinfo" in flags
    assert "sm_90" not in flags and "sm_80" not in flags
    with pytest.raises(build.KernelBuildError):
        build._compile("no_such_kernel")
