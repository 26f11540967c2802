"""The library's host side tested in C++ against its own public header, without a GPU: tests/cpp/host_tests.cpp is built
against the library and each of its cases becomes one test here (the cache's bookkeeping, the arena plan, the generation
loop's decisions with a stand-in stepper, the tokenizer and the streamer, the JSON reader, the registries)."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_exe = None


def _build(workdir: str) -> str:
    global _exe
    if _exe is None:
        from velomind_b200.kernels import library
        main = library.build()
        bdir = os.path.dirname(main)
        out = os.path.join(workdir, "host_tests")
        cuda_inc = os.path.join(os.path.dirname(os.path.dirname(library._nvcc())), "include")
        cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", library.INCLUDE, "-I", cuda_inc, os.path.join(HERE, "cpp", "host_tests.cpp"), "-o", out,
               "-L", bdir, "-l:" + os.path.basename(main), f"-Wl,-rpath,{bdir}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        _exe = out
    return _exe


@pytest.fixture(scope="session")
def host_tests(tmp_path_factory):
    return _build(str(tmp_path_factory.mktemp("host_tests")))


CASES = ["free_list_never_loses_or_doubles", "slots_and_pages_come_back", "groups_with_different_needs_have_their_own_storage",
         "arena_plan_packs_by_liveness", "loop_unequal_prompts_stop_tokens_and_early_ends", "loop_runs_batch_after_batch_and_reuses_slots",
         "batches_are_cut_by_pages_and_slots", "loop_closes_slots_when_a_step_fails", "loop_with_queued_decode_runs_gives_the_same_tokens",
         "pretokenizer_pieces", "bpe_round_trip_and_special_ids", "streamer_emits_deltas_and_waits_for_whole_characters",
         "json_reads_and_writes", "parts_and_architectures_are_looked_up_by_name"]


def test_every_case_is_listed(host_tests):
    listed = subprocess.run([host_tests, "--list"], capture_output=True, text=True, timeout=60).stdout.split()
    assert sorted(listed) == sorted(CASES)


@pytest.mark.parametrize("case", CASES)
def test_host(host_tests, case):
    r = subprocess.run([host_tests, case], capture_output=True, text=True, timeout=120, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and r.stdout.strip() == f"ok {case}", r.stdout + r.stderr
