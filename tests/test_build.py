"""The extension builder's rules that need no GPU: no compiler and no built library is an error."""

import pytest

import turboserve_b200.ops.build as build


def test_a_missing_compiler_is_an_error_not_a_fallback(tmp_path, monkeypatch):
    def no_compiler():
        raise build.ExtensionBuildError("nvcc was not found (test)")

    monkeypatch.setenv("TURBOSERVE_B200_BUILD_DIR", str(tmp_path))
    monkeypatch.setattr(build, "find_nvcc", no_compiler)
    monkeypatch.setattr(build, "_loaded", {})
    for name in build.LIBRARIES:
        with pytest.raises(build.ExtensionBuildError, match="nvcc was not found"):
            build.load_library(name, verbose=False)
    assert not list(tmp_path.iterdir())


def test_every_library_names_a_source_that_exists():
    for name, (source, _) in build.LIBRARIES.items():
        assert (build.CSRC_DIR / source).is_file(), name


def test_the_file_name_changes_with_the_flags(monkeypatch, tmp_path):
    monkeypatch.setenv("TURBOSERVE_B200_BUILD_DIR", str(tmp_path))
    plain, _, _ = build.library_path("layer_ops")
    other, command, _ = build.library_path("layer_ops", defines=("TS_SOMETHING=1",))
    assert plain != other and "-DTS_SOMETHING=1" in command and plain.parent == tmp_path
