// Data-parallel optimizer steps written in the CoCoNet DSL, in the three
// schedules of the CoCoNet paper:
//   AR_C          AllReduce, then the update on every element on every rank
//   RS_C_AG       ReduceScatter, update of the rank's slice, AllGather
//   fuse_RS_C_AG  the same, fused into one kernel (the B200 runtime's path)
// usage: optimizers <sgd|adam|lamb|nesterov|adam_derived|adam_mixed> <AR_C|RS_C_AG|fuse_RS_C_AG> [output.cu]
//        optimizers <sgd|adam|lamb|nesterov> autotune [output directory]
//          (the program written once with AllReduce; the three schedules are derived)
#include <dsl.hpp>
#include <pipeline.hpp>

#include <iostream>
#include <string>

using namespace ACCCDSL;

// `autotune`: the program as written with AllReduce; the Autotuner derives and
// emits the three schedules into the directory `dir`.
static void derive_all(Pipeline &pipeline, std::vector<Tensor> state, const std::string &dir) {
  Autotuner tuner;
  tuner.setOutputDir(dir);
  tuner.autotune(pipeline, state);
  for (const std::string &f : tuner.emitted()) std::cout << f << std::endl;
}

static void sgd(const std::string &schedule, const std::string &out) {
  Variable N(Int32, "N");
  Variable lr(Float32, "lr");
  Tensor g(Float32, N, Local, "g");
  Tensor w(Float32, N, Replicated, "w");
  if (schedule == "AR_C" || schedule == "autotune") {
    Stage gsum = AllReduce(Summation, g);
    Stage wnew = Update(w, w - lr * gsum);
    Pipeline pipeline("sgd", {g, w, lr}, {wnew});
    if (schedule == "autotune") return derive_all(pipeline, {}, out);
    pipeline.codegen(out);
    return;
  }
  Stage gslice = ReduceScatter(Summation, g);
  Stage wslice = Scatter(w) - lr * gslice;
  Stage wnew = Update(w, AllGather(wslice));
  Pipeline pipeline("sgd", {g, w, lr}, {wnew});
  if (schedule == "fuse_RS_C_AG") pipeline.fuse({gslice, wslice, wnew});
  pipeline.codegen(out);
}

static void adam(const std::string &schedule, const std::string &out) {
  Variable N(Int32, "N");
  Variable lr(Float32, "lr"), beta1(Float32, "beta1"), beta2(Float32, "beta2");
  Tensor g(Float32, N, Local, "g");
  Tensor w(Float32, N, Replicated, "w");
  const bool sliced = schedule != "AR_C" && schedule != "autotune";
  Tensor m(Float32, N, sliced ? Sliced : Replicated, "m");
  Tensor v(Float32, N, sliced ? Sliced : Replicated, "v");
  Stage gred = sliced ? Stage(ReduceScatter(Summation, g)) : Stage(AllReduce(Summation, g));
  Stage mnew = Update(m, beta1 * m + (1 - beta1) * gred);
  Stage vnew = Update(v, beta2 * v + (1 - beta2) * gred * gred);
  Stage mhat = mnew / beta1;
  Stage vhat = vnew / beta2;
  if (!sliced) {
    Stage wnew = Update(w, w - lr * mhat / vhat);
    Pipeline pipeline("adam", {g, w, m, v, lr, beta1, beta2}, {mnew, vnew, wnew});
    if (schedule == "autotune") return derive_all(pipeline, {m, v}, out);
    pipeline.fuse({mnew, vnew, mhat, vhat, wnew});
    pipeline.codegen(out);
    return;
  }
  Stage wslice = Scatter(w) - lr * mhat / vhat;
  Stage wnew = Update(w, AllGather(wslice));
  Pipeline pipeline("adam", {g, w, m, v, lr, beta1, beta2}, {mnew, vnew, wnew});
  if (schedule == "fuse_RS_C_AG")
    pipeline.fuse({gred, mnew, vnew, mhat, vhat, wslice, wnew});
  else
    pipeline.fuse({mnew, vnew, mhat, vhat, wslice});
  pipeline.codegen(out);
}

static void lamb(const std::string &schedule, const std::string &out) {
  Variable N(Int32, "N");
  Variable lr(Float32, "lr"), beta1(Float32, "beta1"), beta2(Float32, "beta2");
  Variable decay(Float32, "decay");
  Tensor g(Float32, N, Local, "g");
  Tensor w(Float32, N, Replicated, "w");
  const bool sliced = schedule != "AR_C" && schedule != "autotune";
  Tensor m(Float32, N, sliced ? Sliced : Replicated, "m");
  Tensor v(Float32, N, sliced ? Sliced : Replicated, "v");
  Stage gred = sliced ? Stage(ReduceScatter(Summation, g)) : Stage(AllReduce(Summation, g));
  Stage mnew = Update(m, beta1 * m + (1.0 - beta1) * gred);
  Stage vnew = Update(v, beta2 * v + (1.0 - beta2) * gred * gred);
  Stage mhat = mnew / (1.0 - beta1);
  Stage vhat = vnew / (1.0 - beta2);
  Stage r = mhat / Sqrt(vhat) + decay * w;
  Stage rnorm = Norm(r);
  Stage wnorm = Norm(w);
  Stage wstep = w - lr * (wnorm / rnorm) * r;
  if (!sliced) {
    Stage wnew = Update(w, wstep);
    Pipeline pipeline("lamb", {g, w, m, v, lr, beta1, beta2, decay}, {wnew});
    if (schedule == "autotune") return derive_all(pipeline, {m, v}, out);
    pipeline.fuse({mnew, vnew, mhat, vhat, r, rnorm, wnorm, wstep, wnew});
    pipeline.codegen(out);
    return;
  }
  Stage wnew = Update(w, AllGather(wstep));
  Pipeline pipeline("lamb", {g, w, m, v, lr, beta1, beta2, decay}, {wnew});
  if (schedule == "fuse_RS_C_AG")
    pipeline.fuse({gred, mnew, vnew, mhat, vhat, r, rnorm, wnorm, wstep, wnew});
  else
    pipeline.fuse({mnew, vnew, mhat, vhat, r, rnorm, wnorm, wstep});
  pipeline.codegen(out);
}

// Mixed-precision Adam: fp16 gradients with a loss scale, fp32 master weights
// that every rank keeps for its own slice only, fp32 Sliced moments, and the
// fp16 weights the model computes with, gathered to all ranks.  The fused
// schedule becomes ONE cocoFusedAdam call with the fp16 copy as its gathered
// output (what the reference's hook hard-codes as `(half*)g, w, (half*)w`,
// src/codegen.cpp:1910).
static void adam_mixed(const std::string &schedule, const std::string &out) {
  if (schedule == "AR_C" || schedule == "autotune") {
    std::cout << "adam_mixed is written on slices: RS_C_AG or fuse_RS_C_AG" << std::endl;
    exit(1);
  }
  Variable N(Int32, "N");
  Variable lr(Float32, "lr"), beta1(Float32, "beta1"), beta2(Float32, "beta2");
  Variable inv_scale(Float32, "inv_scale");
  Tensor g(Float16, N, Local, "g");
  Tensor w(Float32, N, Sliced, "w");
  Tensor wh(Float16, N, Replicated, "wh");
  Tensor m(Float32, N, Sliced, "m");
  Tensor v(Float32, N, Sliced, "v");
  Stage gred = ReduceScatter(Summation, g);
  Stage gs = Cast(Float32, gred) * inv_scale;
  Stage mnew = Update(m, beta1 * m + (1 - beta1) * gs);
  Stage vnew = Update(v, beta2 * v + (1 - beta2) * gs * gs);
  Stage mhat = mnew / beta1;
  Stage vhat = vnew / beta2;
  Stage wnew = Update(w, w - lr * mhat / vhat);
  Stage wcast = Cast(Float16, wnew);
  Stage whnew = Update(wh, AllGather(wcast));
  Pipeline pipeline("adam_mixed", {g, w, wh, m, v, lr, beta1, beta2, inv_scale}, {mnew, vnew, wnew, whnew});
  if (schedule == "fuse_RS_C_AG")
    pipeline.fuse({gred, gs, mnew, vnew, mhat, vhat, wnew, wcast, whnew});
  else
    pipeline.fuse({gs, mnew, vnew, mhat, vhat, wnew, wcast});
  pipeline.codegen(out);
}

// Adam written ONCE, as AllReduce + update on every element, and then scheduled
// with CoCoNet's transformations instead of being rewritten by hand:
//   split    AllReduce -> ReduceScatter + AllGather
//   reorder  the update moves below the AllGather and runs on the slice
//   asSlice  the moments are kept as Sliced tensors
//   fuse     everything into one kernel
// `schedule` selects how far the derivation goes.
static void adam_derived(const std::string &schedule, const std::string &out) {
  Variable N(Int32, "N");
  Variable lr(Float32, "lr"), beta1(Float32, "beta1"), beta2(Float32, "beta2");
  Tensor g(Float32, N, Local, "g");
  Tensor w(Float32, N, Replicated, "w");
  Tensor m(Float32, N, Replicated, "m");
  Tensor v(Float32, N, Replicated, "v");
  Stage gsum = AllReduce(Summation, g);
  Stage mnew = Update(m, beta1 * m + (1 - beta1) * gsum);
  Stage vnew = Update(v, beta2 * v + (1 - beta2) * gsum * gsum);
  Stage mhat = mnew / beta1;
  Stage vhat = vnew / beta2;
  Stage wnew = Update(w, w - lr * mhat / vhat);
  Pipeline pipeline("adam", {g, w, m, v, lr, beta1, beta2}, {mnew, vnew, wnew});
  if (schedule == "AR_C") {
    pipeline.fuse({mnew, vnew, mhat, vhat, wnew});
    pipeline.codegen(out);
    return;
  }
  std::pair<Stage, Stage> rsag = pipeline.split(gsum, AllReduceRSAG);
  ReorderedStages re = pipeline.reorder({mnew, vnew, mhat, vhat, wnew}, rsag.second);
  pipeline.asSlice({m, v});
  if (schedule == "fuse_RS_C_AG") {
    std::vector<Stage> all = {rsag.first};
    all.insert(all.end(), re.compStages.begin(), re.compStages.end());
    all.insert(all.end(), re.allGatherStages.begin(), re.allGatherStages.end());
    pipeline.fuse(all);
  } else {
    // after asSlice the two moment updates are plain slice computations again
    std::vector<Stage> comp = re.compStages;
    comp.push_back(mnew);
    comp.push_back(vnew);
    pipeline.fuse(comp);
  }
  pipeline.codegen(out);
}

// SGD with Nesterov momentum: not one of the rules the runtime ships a kernel
// for, so the fused schedule compiles its arithmetic into a device functor for
// the generic fused kernel (include/coconet_fused_generic.cuh).
static void nesterov(const std::string &schedule, const std::string &out) {
  Variable N(Int32, "N");
  Variable lr(Float32, "lr"), mu(Float32, "mu");
  Tensor g(Float32, N, Local, "g");
  Tensor w(Float32, N, Replicated, "w");
  const bool sliced = schedule != "AR_C" && schedule != "autotune";
  Tensor mom(Float32, N, sliced ? Sliced : Replicated, "mom");
  if (!sliced) {
    Stage gsum = AllReduce(Summation, g);
    Stage mnew = Update(mom, mu * mom + gsum);
    Stage wnew = Update(w, w - lr * (gsum + mu * mnew));
    Pipeline pipeline("nesterov", {g, w, mom, lr, mu}, {mnew, wnew});
    if (schedule == "autotune") return derive_all(pipeline, {mom}, out);
    pipeline.fuse({mnew, wnew});
    pipeline.codegen(out);
    return;
  }
  Stage gslice = ReduceScatter(Summation, g);
  Stage mnew = Update(mom, mu * mom + gslice);
  Stage wslice = Scatter(w) - lr * (gslice + mu * mnew);
  Stage wnew = Update(w, AllGather(wslice));
  Pipeline pipeline("nesterov", {g, w, mom, lr, mu}, {mnew, wnew});
  if (schedule == "fuse_RS_C_AG")
    pipeline.fuse({gslice, mnew, wslice, wnew});
  else
    pipeline.fuse({mnew, wslice});
  pipeline.codegen(out);
}

int main(int argc, char **argv) {
  if (argc < 3) {
    std::cout << "usage: " << argv[0] << " <sgd|adam|lamb|nesterov> <AR_C|RS_C_AG|fuse_RS_C_AG> [out.cu]\n";
    return 1;
  }
  const std::string opt = argv[1], schedule = argv[2];
  if (schedule != "AR_C" && schedule != "RS_C_AG" && schedule != "fuse_RS_C_AG" && schedule != "autotune") {
    std::cout << "Invalid schedule" << std::endl;
    return 1;
  }
  // for `autotune` the third argument is the output DIRECTORY (default: the current one)
  const std::string out = argc > 3 ? argv[3] : schedule == "autotune" ? "." : opt + "-" + schedule + ".cu";
  if (opt == "sgd") sgd(schedule, out);
  else if (opt == "adam") adam(schedule, out);
  else if (opt == "lamb") lamb(schedule, out);
  else if (opt == "nesterov") nesterov(schedule, out);
  else if (opt == "adam_derived") adam_derived(schedule, out);
  else if (opt == "adam_mixed") adam_mixed(schedule, out);
  else { std::cout << "Invalid optimizer" << std::endl; return 1; }
  return 0;
}
