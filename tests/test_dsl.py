"""CPU tests of the DSL front end and the emitter: the library builds, the
reference's own example programs compile against it unchanged (when the
reference tree is present), every schedule emits, fused groups are recognised
from what they compute, fusion validity, and emitted programs compile with
nvcc for sm_100a."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DSL = os.path.join(ROOT, "coconet_b200", "dsl")
# the reference tree, when there is one: COCONET_REFERENCE, else a directory
# named "reference" beside the repository
REF = os.environ.get("COCONET_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


@pytest.fixture(scope="module")
def dsl_build():
    subprocess.check_call(["make", "-C", DSL, "-s"])
    return os.path.join(DSL, "build")


def _gen(build, opt, schedule, tmp_path):
    out = str(tmp_path / f"{opt}-{schedule}.cu")
    subprocess.check_call([os.path.join(build, "optimizers"), opt, schedule, out])
    return open(out).read()


@pytest.mark.parametrize("opt,call", [
    ("sgd", "cocoFusedSGD(comm, g, cocoFloat32, w, NULL, cocoFloat16, N, lr, 1.0f, stream)"),
    ("adam", "cocoFusedAdam(comm, g, cocoFloat32, w, NULL, cocoFloat16, m, v, N, lr, beta1, beta2, "
             "0.0f, iter, 1.0f, cocoVariantDsl, stream)"),
    ("lamb", "cocoFusedLAMB(comm, g, cocoFloat32, w, NULL, cocoFloat16, m, v, N, lr, beta1, beta2, "
             "0.0f, decay, iter, 1.0f, cocoVariantDsl, 0, stream)"),
    # mixed precision: fp16 gradients, the loss-scale Variable as the gradient scale, the fp32
    # master Sliced (indexed by global element inside the slice), the fp16 copy gathered
    ("adam_mixed", "cocoFusedAdam(comm, g, cocoFloat16, (w - (size_t)DIVUP(N, comm_size) * rank), wh, "
                   "cocoFloat16, m, v, N, lr, beta1, beta2, 0.0f, iter, inv_scale, cocoVariantDsl, stream)"),
])
def test_fused_schedule_emits_one_runtime_call(dsl_build, tmp_path, opt, call):
    text = _gen(dsl_build, opt, "fuse_RS_C_AG", tmp_path)
    assert call in text
    assert "nccl" not in text and "mpi" not in text.lower()
    assert "__global__" not in text            # no separate kernel: everything is in the fused step
    assert "FusedAllReduce: %f, Total: %f}" in text   # the reference's report line
    assert "cocoCommInitRank(&comm, comm_size, rank, NULL)" in text


@pytest.mark.parametrize("opt", ["sgd", "adam", "lamb"])
@pytest.mark.parametrize("schedule", ["AR_C", "RS_C_AG"])
def test_unfused_schedules_emit_stock_collectives_and_kernels(dsl_build, tmp_path, opt, schedule):
    text = _gen(dsl_build, opt, schedule, tmp_path)
    assert "cocoFused" not in text
    assert "__global__ void binOpFunc0" in text
    assert "nccl" not in text                      # the runtime's own collectives: no NCCL, no MPI
    if schedule == "AR_C":
        assert "cocoAllReduce(comm, g, N, stream)" in text
    else:
        assert "cocoReduceScatter(comm, g, g + (size_t)DIVUP(N, comm_size) * rank, N, stream)" in text
        assert "cocoAllGather(comm, " in text
        assert "m[i0]" in text or opt == "sgd"     # Sliced state is indexed from the slice start
    if opt == "lamb":
        assert text.count("coconetSumSquares<<<") == 2


def test_dsl_cases(dsl_build, tmp_path):
    exe = str(tmp_path / "dsl_cases")
    subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(DSL, "include"),
                           os.path.join(ROOT, "tests", "dsl_cases.cpp"),
                           os.path.join(dsl_build, "libcoconet_dsl.a"), "-o", exe])
    out = dict(line.split(": ", 1) for line in subprocess.check_output([exe], text=True).splitlines())
    assert out["base"] == "1" and out["three"] == "1"
    assert out["unused"] == "0"
    assert out["cycle"] == "0" and out["cycle_reason"] == "1" and out["cycle_all"] == "1"
    assert int(out["groups_after"]) == int(out["groups_before"]) - 1
    assert out["sgd_commuted"] == "SGD lr=''"
    assert out["adam_permuted"] == "Adam m=first v=second b1=b1 b2=b2 lr=lr"
    assert out["momentum"] == "Unknown"


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "examples", "adam")),
                    reason="reference tree not present")
@pytest.mark.parametrize("ex", ["sgd", "adam", "lamb"])
def test_reference_example_programs_are_a_drop_in(dsl_build, tmp_path, ex):
    # the reference's own DSL programs, compiled unchanged from where they lie
    exe = str(tmp_path / ex)
    subprocess.check_call(["g++", "-std=c++17", "-w", "-I", os.path.join(DSL, "include"),
                           os.path.join(REF, "examples", ex, f"{ex}.cpp"),
                           os.path.join(dsl_build, "libcoconet_dsl.a"), "-o", exe])
    for schedule, suffix in [("AR_C", "ar-c"), ("RS_C_AG", "rs-c-ag"), ("fuse_RS_C_AG", "fuse-rs-c-ag")]:
        subprocess.check_call([exe, schedule], cwd=tmp_path)
        text = open(tmp_path / f"{ex}-{suffix}.cu").read()
        assert ("cocoFused" in text) == (schedule == "fuse_RS_C_AG")
    fused = open(tmp_path / f"{ex}-fuse-rs-c-ag.cu").read()
    want = {"sgd": "cocoFusedSGD(comm, g, cocoFloat32, w, NULL, cocoFloat16, N, lr, 1.0f, stream)",
            # adam.cpp:70 has no learning rate; lamb.cpp names its decay variable "gamma"
            "adam": "m, v, N, 1.0f, beta1, beta2, 0.0f, iter, 1.0f, cocoVariantDsl, stream)",
            "lamb": "m, v, N, lr, beta1, beta2, 0.0f, gamma, iter, 1.0f, cocoVariantDsl, 0, stream)"}[ex]
    assert want in fused
    out = subprocess.run([exe, "fuse(RS_C_AG)"], cwd=tmp_path, capture_output=True, text=True)
    assert "Invalid schedule" in out.stdout     # as the reference (examples/sgd/sgd.cpp:67)


@pytest.mark.parametrize("opt,schedule", [("adam", "fuse_RS_C_AG"), ("lamb", "fuse_RS_C_AG"),
                                          ("lamb", "RS_C_AG"), ("sgd", "AR_C"),
                                          ("adam_mixed", "fuse_RS_C_AG"), ("adam_mixed", "RS_C_AG")])
def test_emitted_programs_compile_for_sm100a(dsl_build, tmp_path, opt, schedule):
    _gen(dsl_build, opt, schedule, tmp_path)
    src = str(tmp_path / f"{opt}-{schedule}.cu")
    subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                           os.path.join(DSL, "rt"), "-I", os.path.join(ROOT, "include"), "-c", src,
                           "-o", str(tmp_path / "x.o")])


def test_other_update_rules_compile_into_a_device_functor(dsl_build, tmp_path):
    text = _gen(dsl_build, "nesterov", "fuse_RS_C_AG", tmp_path)
    assert '#include "coconet_fused_generic.cuh"' in text
    assert "struct nesterovFused0 {" in text
    assert "mom[i0] = ((mu * mom[i0]) + gsum);" in text
    assert "(w_old - (lr * (gsum + (mu * mom[i0]))))" in text
    assert "cocoFusedGenericPlan(comm, g, cocoFloat32, w, N, 1.0f, stream, &plan)" in text
    assert "cocoLaunchGenericFused<float>(plan, f, stream)" in text
    assert "cocoMemAlloc(comm, (void**)&g" in text and "cocoMemAlloc(comm, (void**)&w" in text
    subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                           os.path.join(DSL, "rt"), "-I", os.path.join(ROOT, "include"), "-c",
                           str(tmp_path / "nesterov-fuse_RS_C_AG.cu"), "-o", str(tmp_path / "n.o")])


def test_unrecognised_fused_group_is_an_error(dsl_build, tmp_path):
    prog = tmp_path / "bad.cpp"
    prog.write_text('''
#include <dsl.hpp>
#include <pipeline.hpp>
using namespace ACCCDSL;
int main() {
  Variable N(Int32, "N"); Variable lr(Float32, "lr");
  Tensor g(Float32, N, Local, "g"); Tensor w(Float32, N, Replicated, "w");
  Stage gs = ReduceScatter(Summation, g);
  Stage nrm = Norm(gs);                    // a global norm that is not LAMB's
  Stage ws = Scatter(w) - lr * gs / nrm;
  Stage wn = Update(w, AllGather(ws));
  Pipeline p("odd", {g, w, lr}, {wn});
  p.fuse({gs, nrm, ws, wn});
  p.codegen("odd.cu");
}''')
    exe = str(tmp_path / "bad")
    subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(DSL, "include"), str(prog),
                           os.path.join(dsl_build, "libcoconet_dsl.a"), "-o", exe])
    r = subprocess.run([exe], cwd=tmp_path, capture_output=True, text=True)
    assert r.returncode == 2 and "is not a ReduceScatter -> SGD | Adam | LAMB" in r.stderr
    assert "it contains a Norm" in r.stderr


ADAM_CALL = ("cocoFusedAdam(comm, g, cocoFloat32, w, NULL, cocoFloat16, m, v, N, lr, beta1, beta2, "
             "0.0f, iter, 1.0f, cocoVariantDsl, stream)")


def test_schedules_derived_by_split_reorder_asslice(dsl_build, tmp_path):
    """One Adam program written as AllReduce + computation; the other two
    schedules are derived from it (reference: src/pipeline.cpp:851-902 split,
    661-843 reorder, 471-587 asSlice) and must emit what the hand-written
    schedules emit."""
    ar = _gen(dsl_build, "adam_derived", "AR_C", tmp_path)
    assert "cocoAllReduce(comm, g, N, stream)" in ar and "cocoFused" not in ar
    rs = _gen(dsl_build, "adam_derived", "RS_C_AG", tmp_path)
    assert "cocoReduceScatter(comm, g, g + (size_t)DIVUP(N, comm_size) * rank, N, stream)" in rs
    assert "cocoAllGather(comm, " in rs and ", w, N, stream)" in rs
    assert "m[i0] = " in rs and "v[i0] = " in rs           # asSlice: the moments live on the slice
    assert "w[DIVUP(N, comm_size) * rank + i0]" in rs      # the weight is still whole
    assert rs.count("__global__") == 1                     # the slice computation is one kernel
    fused = _gen(dsl_build, "adam_derived", "fuse_RS_C_AG", tmp_path)
    assert ADAM_CALL in fused and "__global__" not in fused
    assert ADAM_CALL in _gen(dsl_build, "adam", "fuse_RS_C_AG", tmp_path)
    for sched in ("RS_C_AG", "fuse_RS_C_AG"):
        subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                               os.path.join(DSL, "rt"), "-I", os.path.join(ROOT, "include"), "-c",
                               str(tmp_path / f"adam_derived-{sched}.cu"), "-o", str(tmp_path / "d.o")])


def _run_dsl_program(tmp_path, body):
    prog = tmp_path / "t.cpp"
    prog.write_text('#include <dsl.hpp>\n#include <pipeline.hpp>\n#include <iostream>\n'
                    'using namespace ACCCDSL;\nint main() {\n'
                    '  Variable N(Int32, "N"); Variable lr(Float32, "lr");\n'
                    '  Tensor g(Float32, N, Local, "g"); Tensor w(Float32, N, Replicated, "w");\n'
                    '  Tensor m(Float32, N, Replicated, "m");\n' + body + '\n  return 0;\n}\n')
    exe = str(tmp_path / "t")
    subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(DSL, "include"), str(prog),
                           os.path.join(DSL, "build", "libcoconet_dsl.a"), "-o", exe])
    return subprocess.run([exe], cwd=tmp_path, capture_output=True, text=True)


def test_transformations_refuse_what_would_change_the_result(dsl_build, tmp_path):
    # split of something that is not an AllReduce
    out = _run_dsl_program(tmp_path, '''
  Stage s = AllReduce(Summation, g); Stage wn = Update(w, w - lr * s);
  Pipeline p("p", {g, w, lr}, {wn});
  p.split(wn, AllReduceRSAG);''')
    assert out.returncode != 0 and "not an AllReduce" in out.stderr
    # reorder that leaves a consumer of the gathered value above the AllGather
    out = _run_dsl_program(tmp_path, '''
  Stage s = AllReduce(Summation, g); Stage mn = Update(m, m + s); Stage wn = Update(w, w - lr * s);
  Pipeline p("p", {g, w, m, lr}, {mn, wn});
  auto rsag = p.split(s, AllReduceRSAG);
  p.reorder({wn}, rsag.second);''')
    assert out.returncode != 0 and "also uses the AllGather" in out.stderr
    # a Norm moves too: it is the norm of the whole tensor, gathered or in slices
    out = _run_dsl_program(tmp_path, '''
  Stage s = AllReduce(Summation, g); Stage u = lr * s; Stage nrm = Norm(u);
  Stage wn = Update(w, w - u / nrm);
  Pipeline p("p", {g, w, lr}, {wn});
  auto rsag = p.split(s, AllReduceRSAG);
  p.reorder({u, nrm, wn}, rsag.second);
  p.codegen("norm.cu");''')
    assert out.returncode == 0, out.stderr
    assert "coconetSumOverRanks" in (tmp_path / "norm.cu").read_text()   # per-rank partial sums
    # ... but a stage that contains a collective does not
    out = _run_dsl_program(tmp_path, '''
  Tensor g2(Float32, N, Local, "g2");
  Stage s = AllReduce(Summation, g); Stage wn = Update(w, w - lr * s * AllReduce(Summation, g2));
  Pipeline p("p", {g, g2, w, lr}, {wn});
  auto rsag = p.split(s, AllReduceRSAG);
  p.reorder({wn}, rsag.second);''')
    assert out.returncode != 0 and "contains a collective" in out.stderr
    # asSlice of a tensor that a stage still computes on whole
    out = _run_dsl_program(tmp_path, '''
  Stage s = AllReduce(Summation, g); Stage mn = Update(m, m + s); Stage wn = Update(w, w - lr * mn);
  Pipeline p("p", {g, w, m, lr}, {mn, wn});
  p.asSlice(m);''')
    assert out.returncode != 0 and "reorder it below the AllGather first" in out.stderr
    # the legal sequence: every stage moves, then the state becomes a slice
    out = _run_dsl_program(tmp_path, '''
  Stage s = AllReduce(Summation, g); Stage mn = Update(m, m + s); Stage wn = Update(w, w - lr * mn);
  Pipeline p("p", {g, w, m, lr}, {mn, wn});
  auto rsag = p.split(s, AllReduceRSAG);
  auto re = p.reorder({mn, wn}, rsag.second);
  p.asSlice(m);
  std::cout << re.compStages.size() << " " << re.allGatherStages.size() << " "
            << (m.layout() == Sliced) << (w.layout() == Replicated) << std::endl;
  p.codegen("seq.cu");''')
    assert out.returncode == 0, out.stderr
    assert out.stdout.split()[:3] == ["2", "2", "11"]
    text = (tmp_path / "seq.cu").read_text()
    assert "cocoReduceScatter(" in text and text.count("cocoAllGather(") == 1


@pytest.mark.parametrize("opt", ["sgd", "adam", "lamb", "nesterov"])
def test_autotuner_derives_the_three_schedules_from_the_allreduce_program(dsl_build, tmp_path, opt):
    """`Autotuner::autotune(pipeline, canSlice)` (reference surface:
    src/pipeline.hpp:675-684) on a program written once with AllReduce: three
    programs come out, the fused one makes the same runtime call as the
    hand-written fused schedule, the unfused ones use the runtime's collectives,
    and all compile."""
    out = subprocess.run([os.path.join(dsl_build, "optimizers"), opt, "autotune", str(tmp_path)],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    files = out.stdout.split()
    assert [os.path.basename(f) for f in files] == [f"{opt}-{s}.cu" for s in
                                                    ("AR_C", "RS_C_AG", "fuse_RS_C_AG")]
    ar, rs, fused = (open(f).read() for f in files)
    assert "cocoAllReduce(comm, g, N, stream)" in ar and "cocoFused" not in ar
    assert "cocoReduceScatter(comm, g, g + (size_t)DIVUP(N, comm_size) * rank, N, stream)" in rs
    assert rs.count("cocoAllGather(comm, ") == 1 and "cocoFused" not in rs
    (tmp_path / "hand").mkdir()
    hand = _gen(dsl_build, opt, "fuse_RS_C_AG", tmp_path / "hand")
    call = [ln.strip() for ln in hand.splitlines() if "COCOCHECK(cocoFused" in ln]
    assert call and all(c in fused for c in call)          # the same fused call(s), argument for argument
    if opt != "sgd":
        assert "m[i0] = " in rs or "mom[i0] = " in rs      # the state lives on the slice
    if opt == "lamb":
        assert rs.count("coconetSumSquares<<<") == 2 and "coconetSumOverRanks" in rs
    for f in files:
        subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                               os.path.join(DSL, "rt"), "-I", os.path.join(ROOT, "include"), "-c", f,
                               "-o", str(tmp_path / "a.o")])


def test_autotuner_refuses_programs_it_cannot_derive_from(dsl_build, tmp_path):
    out = _run_dsl_program(tmp_path, '''
  Stage s = ReduceScatter(Summation, g); Stage wn = Update(w, AllGather(Scatter(w) - lr * s));
  Pipeline p("p", {g, w, lr}, {wn});
  Autotuner().autotune(p);''')
    assert out.returncode != 0 and "write the pipeline with AllReduce only" in out.stderr
    out = _run_dsl_program(tmp_path, '''
  Stage wn = Update(w, w - lr * w);
  Pipeline p("p", {g, w, lr}, {wn});
  Autotuner().autotune(p);''')
    assert out.returncode != 0 and "no AllReduce" in out.stderr


def test_autotuner_on_a_program_with_a_gradient_norm(dsl_build, tmp_path):
    # w -= lr * gsum / ||gsum||: the Norm reads the collective's in-place result (whole
    # buffer after AllReduce, the rank's slice after ReduceScatter); no fused schedule,
    # because a global norm inside one kernel exists for LAMB only
    out = _run_dsl_program(tmp_path, '''
  Stage s = AllReduce(Summation, g); Stage nrm = Norm(s); Stage wn = Update(w, w - lr * s / nrm);
  Pipeline p("clip", {g, w, lr}, {wn});
  Autotuner t; t.autotune(p);
  for (const std::string &f : t.emitted()) std::cout << f << std::endl;''')
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["./clip-AR_C.cu", "./clip-RS_C_AG.cu"]
    assert "the fused schedule of 'clip' is not emitted" in out.stderr
    ar, rs = (tmp_path / "clip-AR_C.cu").read_text(), (tmp_path / "clip-RS_C_AG.cu").read_text()
    assert "coconetSumSquares<<<coconetBlocks(N), 256, 0, stream>>>(g, N, " in ar
    assert "(g + (size_t)DIVUP(N, comm_size) * rank), coconetSliceLen(N, comm_size, rank), " in rs
    assert "coconetSumOverRanks(comm, " in rs and "coconetSumOverRanks" not in ar
    for f in ("clip-AR_C.cu", "clip-RS_C_AG.cu"):
        subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                               os.path.join(DSL, "rt"), "-I", os.path.join(ROOT, "include"), "-c",
                               str(tmp_path / f), "-o", str(tmp_path / "c.o")])
