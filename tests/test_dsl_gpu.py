"""Programs emitted by the DSL, built with nvcc and run on the GPU as plain
C++ executables (no Python in the process): each runs one step and compares it
with the host evaluation of the same pipeline that the emitter generated
beside it, then runs its timed loop and prints the reference's report line."""
import os
import re
import subprocess

import pytest

import dsl_build_util as B

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("opt,schedule", [("sgd", "fuse_RS_C_AG"), ("adam", "fuse_RS_C_AG"),
                                          ("lamb", "fuse_RS_C_AG"), ("adam", "RS_C_AG"),
                                          ("lamb", "AR_C"), ("nesterov", "fuse_RS_C_AG"),
                                          ("adam_derived", "RS_C_AG"),
                                          ("adam_derived", "fuse_RS_C_AG"),
                                          ("adam_mixed", "fuse_RS_C_AG"),
                                          ("adam_mixed", "RS_C_AG")])
def test_emitted_program_runs_and_checks_world_1(tmp_path, opt, schedule):
    exe = B.build_program(opt, schedule, str(tmp_path))
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1",
               MASTER_PORT="29877", **B.SCALARS)
    r = subprocess.run([exe, "3", "10", "17", "check"], env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("PASSED") == 7 and "FAILED" not in r.stdout
    lines = re.findall(r"\{SZ: (\d+), Epochs: 3, .*Total: ([0-9.]+)\}", r.stdout)
    assert [int(a) for a, _ in lines] == [1 << k for k in range(10, 17)]
    if schedule == "fuse_RS_C_AG":
        assert "FusedAllReduce:" in r.stdout


def test_measuring_autotuner_ranks_the_schedules():
    from coconet_b200.dsl.autotune import autotune
    res = autotune("adam", gpus=1, log2=22, epochs=5,
                   scalars={"beta1": 0.9, "beta2": 0.999, "lr": 0.01})
    assert [r["schedule"] for r in res["results"]] == ["AR_C", "RS_C_AG", "fuse_RS_C_AG"]
    assert all(r["ms_per_step"] > 0 for r in res["results"])
    assert res["best"] in ("AR_C", "RS_C_AG", "fuse_RS_C_AG")
    # the fused schedule is one stage; the unfused ones report their collectives too
    assert list(res["results"][2]["stages_ms"]) == ["FusedAllReduce"]
    assert "AllReduce" in res["results"][0]["stages_ms"]
