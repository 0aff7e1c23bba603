"""Every bench and kit program imports on a machine without a GPU and explains itself: a tool that
only ever runs on GPU boxes must not hide an import error or a broken argument parser until it
is needed there.  In-process, so the whole list costs seconds."""
import importlib
import inspect
import pkgutil

import pytest

import gpubridge_b200.bench
import gpubridge_b200.kit


def programs():
    found = []
    for package in (gpubridge_b200.bench, gpubridge_b200.kit):
        for info in pkgutil.iter_modules(package.__path__):
            if not info.ispkg and not info.name.startswith("_"):
                found.append(f"{package.__name__}.{info.name}")
    return sorted(found)


PROGRAMS = programs()


def test_the_list_is_not_empty_and_knows_the_main_tools():
    assert len(PROGRAMS) >= 30
    for name in ("bench.bench_all_reduce", "bench.train_dp", "bench.ddp_attribution", "bench.bench_gemm_team",
                 "kit.check", "kit.runbook", "kit.rdma_kit", "kit.gloo_dtypes", "kit.codec_diagnosis"):
        assert f"gpubridge_b200.{name}" in PROGRAMS


@pytest.mark.parametrize("name", PROGRAMS)
def test_a_program_imports_without_a_gpu_and_says_what_it_is(name):
    module = importlib.import_module(name)
    assert (module.__doc__ or "").strip(), f"{name} has no description"
    main = getattr(module, "main", None)
    if main is None:
        return                                                     # a library of helpers, not a program
    parameters = list(inspect.signature(main).parameters)
    if parameters[:1] != ["argv"] or "argparse" not in inspect.getsource(module):
        return                       # reads sys.argv itself, takes its case by name, or reads bare words: not called here
    with pytest.raises(SystemExit) as stopped:
        main(["--help"])
    assert stopped.value.code == 0


def test_help_texts_name_the_program(capsys):
    from gpubridge_b200.bench import bench_all_reduce, bench_gemm_team
    from gpubridge_b200.kit import rdma_kit
    for module in (bench_all_reduce, bench_gemm_team, rdma_kit):
        with pytest.raises(SystemExit):
            module.main(["--help"])
        told = capsys.readouterr().out
        assert "usage:" in told and len(told) > 200


def test_programs_that_read_bare_words_answer_help_instead_of_taking_it_for_a_file(tmp_path, monkeypatch, capsys):
    from gpubridge_b200.kit import baseline_identity, gloo_dtypes, summarize
    monkeypatch.chdir(tmp_path)
    for module in (baseline_identity, gloo_dtypes, summarize):
        assert module.main(["--help"]) == 0
        assert "python -m gpubridge_b200.kit" in capsys.readouterr().out
    assert baseline_identity.main(["--out"]) == 2 and gloo_dtypes.main(["--json"]) == 2 and summarize.main(["--all"]) == 2
    assert list(tmp_path.iterdir()) == []                          # nothing was written under a flag's name
