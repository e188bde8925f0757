"""The reference's own callers and tools on top of libbmb.so, and the file formats either side of the
training step.

  * the six drop-in binaries (oracle/_ref/dropin_*: the reference's gpt.cu, train_gpt.cu, bench.cu and its
    four test programs, compiled unmodified and linked with libbmb.so in place of the reference's
    kernels) must run: the test programs exit 0, the registry harness verifies its entries against its
    own checker and writes its CSV, train_gpt prints the reference's step lines with losses within 2e-3 of
    the reference's own build (oracle/_ref/ref_train_gpt) on the same synthetic text;
  * GPT1 checkpoints (src/train_gpt.cu:175-227) go both ways between this library and the reference's
    train_gpt, bit for bit, and sampling from the same checkpoint gives the same text;
  * bmb_train_gpt, the driver over the C ABI, prints what the reference's Python tools parse
    (tools/plot_training.py:12-13, tools/flash_memory.py:39-41), resumes from optimiser state, and
    kernel_bench.py writes the registry sweep in the harness's CSV columns (src/bench.cu:244).

Skipped when oracle/_ref/ was not built (the reference checkout was absent at build time).
"""
import os
import re
import struct
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
PKG = os.path.join(ROOT, "bare-metal-bard_b200")

# the patterns the reference's tools apply to a training log / an --alloc-only report
STEP_LINE = re.compile(r"^step\s+(\d+)/(\d+)\s+loss\s+([\d.]+)", re.M)             # tools/plot_training.py:12
EVAL_LINE = re.compile(r"\[eval\]\s+step\s+(\d+)\s+val loss\s+([\d.]+)")           # tools/plot_training.py:13
PARAMS = re.compile(r"^params\s+([\d.]+)M", re.M)                                   # tools/flash_memory.py:39
MEM = re.compile(r"^memory\s+([\d.]+) MB forward activations, ([\d.]+) MB", re.M)   # tools/flash_memory.py:40
TOTAL = re.compile(r"^total\s+([\d.]+) GB", re.M)                                   # tools/flash_memory.py:41


def exe(name):
    p = os.path.join(REF_DIR, name)
    if not os.path.exists(p):
        pytest.skip("%s not built (needs the reference checkout at build time)" % name)
    return p


def run(cmd, cwd=None, env=None, timeout=900):
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=cwd, env=dict(os.environ, **(env or {})))
    return r.returncode, r.stdout + r.stderr


@pytest.fixture(scope="module")
def text_file(tmp_path_factory):
    """A few hundred KB of printable bytes with some structure (word-like runs and newlines), standing in for
    the text corpus the reference trains on."""
    rng = np.random.default_rng(7)
    words = ["".join(chr(c) for c in rng.integers(97, 123, rng.integers(2, 9))) for _ in range(400)]
    picks = rng.integers(0, len(words), 60000)
    out, col = [], 0
    for i in picks:
        out.append(words[i])
        col += len(words[i]) + 1
        out.append("\n" if col > 60 else " ")
        col = 0 if col > 60 else col
    d = tmp_path_factory.mktemp("corpus")
    p = d / "input.txt"
    p.write_text("".join(out))
    return str(p)


@pytest.mark.parametrize("name", ["dropin_test_grad", "dropin_test_flash", "dropin_test_ddp", "dropin_test_gemm"])
def test_reference_test_programs_pass_against_libbmb(cuda, name):
    rc, out = run([exe(name)], env={"BMB_MATH": "fp32"})
    assert rc == 0, out[-3000:]


def test_registry_harness_verifies_and_writes_its_csv(cuda, tmp_path):
    csv = tmp_path / "run.csv"
    rc, out = run([exe("dropin_sgemm"), "-k", "1,2,3", "-s", "1024,2048", "--csv", str(csv)])
    assert rc == 0 and "FAIL" not in out, out[-3000:]
    assert out.count(" ok") >= 6, out[-3000:]
    lines = csv.read_text().strip().splitlines()
    assert lines[0] == "kernel_id,kernel,size,gflops_best,gflops_median,cublas_gflops_best,pct_of_cublas"
    assert len(lines) == 7 and lines[1].startswith("1,simt_fp32,1024,")
    # the tensor-core flag of the harness (its checker switched to TF32; verification off by its own rule)
    rc, out = run([exe("dropin_sgemm"), "-k", "1,2,3", "-s", "1024,2048", "--tf32"])
    assert rc == 0 and out.count("skipped") == 6, out[-3000:]


def losses_of(out):
    return {int(m.group(1)): float(m.group(3)) for m in STEP_LINE.finditer(out)}


def test_train_gpt_dropin_matches_the_reference_build(cuda, text_file, tmp_path):
    """20 steps of the reference's train_gpt, once built from its own kernels and once linked with libbmb.so:
    same step lines, losses within 2e-3; --alloc-only reports the same memory; a checkpoint saved by either
    loads in the other and samples the same text."""
    args = ["-d", text_file, "-n", "20", "-b", "4", "-t", "64", "-l", "2", "--eval", "20", "--eval-batches", "2",
            "--sample", "0", "--len", "0", "--warmup", "5"]
    ck_ref, ck_bmb = str(tmp_path / "ref.bin"), str(tmp_path / "bmb.bin")
    rc1, out1 = run([exe("ref_train_gpt")] + args + ["--save", ck_ref])
    rc2, out2 = run([exe("dropin_train_gpt")] + args + ["--save", ck_bmb], env={"BMB_MATH": "fp32"})
    assert rc1 == 0 and rc2 == 0, out1[-2000:] + out2[-2000:]
    l1, l2 = losses_of(out1), losses_of(out2)
    assert sorted(l1) == sorted(l2) == [1, 10, 20], (l1, l2)
    assert max(abs(l1[k] - l2[k]) for k in l1) < 2e-3, (l1, l2)
    v1, v2 = EVAL_LINE.search(out1), EVAL_LINE.search(out2)
    assert v1 and v2 and abs(float(v1.group(2)) - float(v2.group(2))) < 2e-3
    # memory report
    rc, a1 = run([exe("ref_train_gpt")] + args + ["--alloc-only"])
    rc2, a2 = run([exe("dropin_train_gpt")] + args + ["--alloc-only"])
    assert rc == 0 and rc2 == 0
    for pat in (PARAMS, MEM, TOTAL):
        assert pat.search(a1).groups() == pat.search(a2).groups()
    # checkpoints cross over, and the same seed draws the same characters from the same file
    texts = {}
    for who in ("ref_train_gpt", "dropin_train_gpt"):
        for ck in (ck_ref, ck_bmb):
            rc, out = run([exe(who), "--load", ck, "--len", "48", "--seed", "5", "-b", "2"], env={"BMB_MATH": "fp32"})
            assert rc == 0 and "loaded" in out, out[-2000:]
            texts[(who, ck)] = out.split("params\n", 1)[1]
    assert texts[("ref_train_gpt", ck_ref)] == texts[("dropin_train_gpt", ck_ref)]
    assert texts[("ref_train_gpt", ck_bmb)] == texts[("dropin_train_gpt", ck_bmb)]


def read_gpt1(path):
    raw = open(path, "rb").read()
    magic, = struct.unpack_from("<i", raw, 0)
    cfg = struct.unpack_from("<6i", raw, 4)
    nvocab, = struct.unpack_from("<i", raw, 28)
    itos = raw[32:32 + nvocab]
    return magic, cfg, itos, raw[32 + nvocab:]


def test_gpt1_checkpoints_both_ways_and_sampling(bmb, cuda, text_file, tmp_path):
    """A checkpoint written by the reference's train_gpt loads here with bit-identical parameters, this
    library's generate() draws the same characters from it as the reference's, and a checkpoint written
    here (with optimiser state appended) loads in the reference's train_gpt."""
    import ctypes as C
    ck_ref = str(tmp_path / "ref.bin")
    rc, out = run([exe("ref_train_gpt"), "-d", text_file, "-n", "10", "-b", "4", "-t", "64", "-l", "2", "--eval", "10",
                   "--eval-batches", "2", "--sample", "0", "--len", "0", "--save", ck_ref])
    assert rc == 0, out[-2000:]
    magic, cfg, itos, body = read_gpt1(ck_ref)
    assert magic == 0x47505431
    lib = bmb.lib()
    hc, nv, has_opt, step = bmb.TrainConfig(), C.c_int(), C.c_int(-1), C.c_int(-1)
    buf = C.create_string_buffer(256)
    bmb.check(lib.bmb_checkpoint_header(ck_ref.encode(), C.byref(hc), C.byref(nv), buf, 256, C.byref(has_opt), C.byref(step)))
    assert (hc.max_seq_len, hc.vocab_size, hc.padded_vocab, hc.n_layer, hc.n_head, hc.n_embd) == cfg
    assert nv.value == len(itos) and buf.raw[:nv.value] == itos and has_opt.value == 0
    model = dict(max_seq_len=cfg[0], vocab_size=cfg[1], padded_vocab=cfg[2], n_layer=cfg[3], n_head=cfg[4], n_embd=cfg[5])
    tr = bmb.Trainer(seed=1, use_flash=1, math=bmb.MATH_FP32, B=2, T=cfg[0], **model)
    tr.load(ck_ref)
    p = np.empty(tr.num_params, np.float32)
    tr.get_params(p)
    assert len(body) == p.nbytes and p.tobytes() == body           # bit-identical parameters
    # same draws as the reference's generate(): seed + 1, temperature 0.8, start at the newline character
    rc, out = run([exe("ref_train_gpt"), "--load", ck_ref, "--len", "48", "--seed", "5", "-b", "2"])
    assert rc == 0, out[-2000:]
    want = out.split("params\n", 1)[1][1:49]                       # the program prints "\n<text>\n"
    toks = tr.generate(itos.index(b"\n"), 48, 6, 0.8)
    got = bytes(itos[t] for t in toks).decode("latin1")
    assert got == want, (got, want)
    # a mismatching trainer refuses the file
    other = bmb.Trainer(seed=1, use_flash=1, math=bmb.MATH_FP32, B=2, T=cfg[0], **dict(model, n_layer=cfg[3] + 1))
    assert lib.bmb_trainer_load(other.h, ck_ref.encode(), 0, None) != 0 and b"layer" in lib.bmb_last_error()
    other.close()
    # write here: the parameters section equals what was loaded; the optimiser section follows it
    rng = np.random.default_rng(0)
    tok = rng.integers(0, cfg[1], (2, cfg[0]), dtype=np.int32)
    tr.upload(tok, tok)
    tr.step(1e-3, 1)
    ck_bmb = str(tmp_path / "bmb.bin")
    tr.save(ck_bmb, itos, with_optimizer_state=True, step=1)
    tr.get_params(p)
    magic2, cfg2, itos2, body2 = read_gpt1(ck_bmb)
    assert (magic2, cfg2, itos2) == (magic, cfg, itos) and body2[:p.nbytes] == p.tobytes()
    assert struct.unpack_from("<2i", body2, p.nbytes) == (0x4F424D42, 1) and len(body2) == 3 * p.nbytes + 8
    bmb.check(lib.bmb_checkpoint_header(ck_bmb.encode(), None, None, None, 0, C.byref(has_opt), C.byref(step)))
    assert has_opt.value == 1 and step.value == 1
    rc, out = run([exe("ref_train_gpt"), "--load", ck_bmb, "--len", "16", "-b", "2"])
    assert rc == 0 and "loaded" in out and ("%d layers" % cfg[3]) in out, out[-2000:]
    # resume: a second trainer restored from the file holds exactly the saved state (writing it out again gives the
    # same bytes: parameters, both AdamW moments, the step) and continues like the first.  The token-embedding
    # gradient is summed with atomics, so the two continuations agree to rounding, not bit for bit -- and AdamW
    # turns a rounding-sized gradient difference into a step-sized parameter difference where the second moment is
    # tiny, so what is compared after the step is the loss, and the parameters to within one learning-rate step.
    tr2 = bmb.Trainer(seed=99, use_flash=1, math=bmb.MATH_FP32, B=2, T=cfg[0], **model)
    assert tr2.load(ck_bmb, optimizer_state=True) == 1
    ck_again = str(tmp_path / "again.bin")
    tr2.save(ck_again, itos, with_optimizer_state=True, step=1)
    assert open(ck_again, "rb").read() == open(ck_bmb, "rb").read()
    losses = []
    for t_ in (tr, tr2):
        t_.upload(tok, tok)
        t_.step(1e-3, 2)
        losses.append(t_.loss())
    q = np.empty_like(p)
    tr.get_params(p)
    tr2.get_params(q)
    assert abs(losses[0] - losses[1]) < 1e-5 and float(np.abs(p - q).max()) <= 2.5e-3
    tr.close()
    tr2.close()


def test_bmb_train_gpt_speaks_the_reference_log_format(cuda, text_file, tmp_path):
    drv = os.path.join(PKG, "bmb_train_gpt")
    assert os.path.exists(drv), "bmb_train_gpt is built with the library (bare-metal-bard_b200/build.py)"
    ck = str(tmp_path / "drv.bin")
    args = ["-d", text_file, "-b", "4", "-t", "64", "-l", "2", "--eval", "20", "--eval-batches", "2", "--sample", "0", "--len", "32",
            "--warmup", "5"]
    rc, out = run([drv] + args + ["-n", "20", "--save", ck, "--save-optimizer"])
    assert rc == 0, out[-3000:]
    steps = losses_of(out)
    assert sorted(steps) == [1, 10, 20] and steps[20] < steps[1]          # it learns the synthetic text
    assert EVAL_LINE.search(out) and "final  train loss" in out and "final sample:" in out
    assert all(p.search(out) for p in (PARAMS, MEM, TOTAL))
    # the reference's own train_gpt on the same text starts from the same initialisation and the same first batch
    rc, ref_out = run([exe("ref_train_gpt")] + args + ["-n", "1", "--len", "0"])
    assert rc == 0 and abs(losses_of(ref_out)[1] - steps[1]) < 2e-3, (ref_out[-1500:], steps)
    # --alloc-only: the report alone; agrees with the reference's for the same model
    rc, a = run([drv] + args + ["--alloc-only"])
    rc2, b = run([exe("ref_train_gpt")] + args + ["--alloc-only"])
    assert rc == 0 and rc2 == 0 and "step" not in a
    assert PARAMS.search(a).groups() == PARAMS.search(b).groups()
    # the checkpoint it wrote loads in the reference's program, and --resume continues from step 20
    rc, out = run([exe("ref_train_gpt"), "--load", ck, "--len", "16", "-b", "2"])
    assert rc == 0 and "loaded" in out, out[-2000:]
    rc, out = run([drv] + args + ["-n", "10", "--resume", ck, "--save", ""])
    assert rc == 0 and "resumed" in out and sorted(losses_of(out)) == [21, 30], out[-3000:]
    # flags the reference's command line lacks: heads, width, synthetic tokens, TF32 arithmetic
    rc, out = run([drv, "--synthetic", "--vocab", "1000", "-b", "4", "-t", "128", "-l", "2", "--heads", "4", "--embd", "256",
                   "--math", "tf32", "-n", "10", "--eval", "0", "--beta2", "0.95", "--len", "0", "--eval-batches", "1"])
    assert rc == 0 and sorted(losses_of(out)) == [1, 10], out[-3000:]


def test_kernel_bench_writes_the_harness_csv(cuda, tmp_path):
    csv = tmp_path / "k.csv"
    for _ in range(2):                       # appends: one header, rows from both runs
        rc, out = run([sys.executable, os.path.join(PKG, "kernel_bench.py"), "registry", "--csv", str(csv), "-s", "512,1024"])
        assert rc == 0, out[-3000:]
    lines = csv.read_text().strip().splitlines()
    assert lines[0] == "kernel_id,kernel,size,gflops_best,gflops_median,cublas_gflops_best,pct_of_cublas"
    assert len(lines) == 1 + 2 * 6
    for ln in lines[1:]:
        f = ln.split(",")
        assert len(f) == 7 and int(f[0]) in (1, 2, 3) and float(f[3]) > 0 and float(f[5]) > 0
