"""The C ABI surface, checked without a GPU: the library loads, exports every
function include/bmb.h declares (and the reference's C++ names), and the
host-only entry points behave."""
import ctypes as C
C_ull = C.c_ulonglong
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "bmb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bmb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(bmb):
    names = declared_functions()
    assert len(names) > 60
    lib = C.CDLL(bmb.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), "libbmb.so does not export %s" % n
        assert n in bmb.SIGNATURES, "python binding table misses %s" % n
    assert set(bmb.SIGNATURES) <= set(names)


def test_reference_cxx_names_are_exported(bmb):
    out = subprocess.run(["nm", "-DC", bmb.LIB_PATH], capture_output=True, text=True).stdout
    for sym in ["gemm(bool, bool, int, int, int, float, float const*, float const*, float, float*, CUstream_st*)",
                "batched_gemm(bool, bool, int, int, int, int, float, float const*, long long, float const*, long long, float, float*, long long, CUstream_st*)",
                "flash_attention_forward(float*, float*, float const*, int, int, int, int)",
                "flash_attention_backward(float*, float*, float const*, float const*, float const*, float const*, int, int, int, int)",
                "flash_attention_forward_cfg(int, float*, float*, float const*, int, int, int, int)",
                "attention_forward(float*, float*, float*, float const*, int, int, int, int)",
                "layernorm_backward(float*, float*, float*, float const*, float const*, float const*, float const*, float const*, int, int)",
                "adamw_update(float*, float*, float*, float*, int, float, float, float, float, float, int, float)",
                "grad_global_norm(float const*, int)", "reduce_mean(float const*, int)",
                "ddp_init(DDP&, int, int const*)", "ddp_allreduce(DDP&, float**, unsigned long)",
                "ddp_timing(DDP const&)", "find_kernel(int)", "KERNELS", "NUM_KERNELS"]:
        assert sym in out, sym


def test_registry_entries(bmb):
    lib = bmb.lib()
    assert lib.bmb_num_kernels() == 3
    want = {1: (b"simt_fp32", 1e-6), 2: (b"tcgen05_tf32", 5e-4), 3: (b"tcgen05_bf16", 8e-3)}
    for kid, (name, tol) in want.items():
        e = lib.bmb_find_kernel(kid).contents
        assert e.name == name and e.tol == tol and e.fn
    assert not lib.bmb_find_kernel(99)


def test_host_only_calls(bmb):
    lib = bmb.lib()
    assert b"sm_100a" in lib.bmb_version()
    assert lib.bmb_flash_num_configs() >= 1 and lib.bmb_flash_num_bwd_configs() >= 1
    assert lib.bmb_flash_config_name(lib.bmb_flash_default_config()) != b"?"
    assert lib.bmb_flash_config_name(999) == b"?"
    assert lib.bmb_set_math_mode(7) != 0 and b"math mode" in lib.bmb_last_error()
    prev = lib.bmb_get_math_mode()
    assert lib.bmb_set_math_mode(bmb.MATH_TF32) == 0 and lib.bmb_get_math_mode() == bmb.MATH_TF32
    lib.bmb_set_math_mode(prev)
    lib.bmb_set_stream(None)
    assert lib.bmb_get_stream() is None


@pytest.mark.parametrize("count,n", [(1, 8), (3, 2), (17, 4), (1000, 3), (65537, 8), (124475904, 8), (5, 8)])
def test_ddp_slices_partition_the_buffer(bmb, count, n):
    lib = bmb.lib()
    off, ln = C.c_size_t(), C.c_size_t()
    covered = 0
    per = (count + n - 1) // n
    for r in range(n):
        assert lib.bmb_ddp_slice(count, n, r, C.byref(off), C.byref(ln)) == 0
        if ln.value:
            assert off.value == covered and ln.value <= per
        covered += ln.value
    assert covered == count
    assert lib.bmb_ddp_slice(10, 2, 2, C.byref(off), C.byref(ln)) != 0


def test_missing_library_fails_loudly(bmb, tmp_path, monkeypatch):
    monkeypatch.setattr(bmb, "_lib", None)
    monkeypatch.setattr(bmb, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(bmb.BmbError, match="no CPU or PyTorch fallback"):
        bmb.lib()


def test_tensorcore_gemm_schedule_covers_every_slice_once(bmb):
    """The tile plan of the tcgen05 GEMM (tile width, whole tiles, tiles shared along K between CTAs),
    replayed on the host for the training step's shapes, odd shapes and random ones, on several SM
    counts: every (tile, K slice) must be computed exactly once."""
    import ctypes as C
    import random
    lib = bmb.lib()
    rng = random.Random(11)
    shapes = [(8192, 2304, 768), (8192, 768, 768), (8192, 3072, 768), (8192, 768, 3072), (8192, 50304, 768),
              (8192, 768, 50304), (3072, 768, 8192), (768, 768, 8192), (50304, 768, 8192), (8192, 8192, 8192),
              (128, 64, 32), (129, 65, 33), (1000, 1000, 1000), (4096, 160, 512),
              # long K, few tiles, operands beyond L2: shared as a whole, in chunk-major order
              (4096, 512, 100000), (2048, 768, 65536), (8192, 256, 40000), (1024, 1024, 30011)]
    shapes += [(rng.randrange(128, 5000), rng.randrange(64, 5000), rng.randrange(32, 5000)) for _ in range(60)]
    shared = 0
    for ctas in (148, 132, 7, 1):
        for (M, N, K) in shapes:
            for flags in (0, bmb.GEMM_NO_SPLIT):
                bm, bn, dp, grid = C.c_int(), C.c_int(), C.c_int(), C.c_int()
                st = lib.bmb_gemm_schedule_check(bmb.MATH_TF32, flags, 1, M, N, K, ctas, C.byref(bm), C.byref(bn), C.byref(dp), C.byref(grid))
                assert st == 0, (M, N, K, ctas, flags, lib.bmb_last_error())
                tiles = -(-M // bm.value) * -(-N // bn.value)
                assert (bm.value, bn.value) in ((128, 64), (128, 128), (128, 192), (128, 256), (256, 256))
                assert 1 <= grid.value <= ctas and 0 <= dp.value <= tiles
                if flags:
                    assert dp.value == tiles
                shared += dp.value < tiles
    assert shared > 20                      # the sweep does exercise shared tiles
    st = lib.bmb_gemm_schedule_check(bmb.MATH_TF32, 0, 96, 1024, 64, 1024, 148, None, None, None, None)   # batched
    assert st == 0, lib.bmb_last_error()
    # the CTA-pair form (256 x 256 tiles handed to pairs), the half-GPU plans of the side-by-side backward
    # products, and the forced tile heights
    for units in (74, 37, 66, 1):
        for (M, N, K) in shapes:
            if M < 256 or N < 256:
                continue
            for flags in (bmb.GEMM_PAIR, bmb.GEMM_PAIR | bmb.GEMM_NO_SPLIT):
                bm, bn, dp, grid = C.c_int(), C.c_int(), C.c_int(), C.c_int()
                st = lib.bmb_gemm_schedule_check(bmb.MATH_TF32, flags, 1, M, N, K, units, C.byref(bm), C.byref(bn), C.byref(dp), C.byref(grid))
                assert st == 0, (M, N, K, units, flags, lib.bmb_last_error())
                assert (bm.value, bn.value) == (256, 256) and 1 <= grid.value <= units
    # a short K whose shared run would be a sizeable part of a CTA's work keeps its tiles whole (dX of the attention
    # projection on half of the SMs: 192 tiles on 74 CTAs end in a partly filled wave instead); a long K is shared
    bm, bn, dp = C.c_int(), C.c_int(), C.c_int()
    assert lib.bmb_gemm_schedule_check(bmb.MATH_TF32, 0, 1, 8192, 768, 768, 74, C.byref(bm), C.byref(bn), C.byref(dp), None) == 0
    assert dp.value == -(-8192 // bm.value) * -(-768 // bn.value)
    assert lib.bmb_gemm_schedule_check(bmb.MATH_TF32, 0, 1, 2304, 768, 8192, 74, C.byref(bm), C.byref(bn), C.byref(dp), None) == 0
    assert dp.value == 0
    for (M, N, K) in shapes[:10]:
        for flags, want in ((bmb.GEMM_TILE_M128 | bmb.GEMM_NO_PAIR, 128), (bmb.GEMM_TILE_M256 | bmb.GEMM_NO_PAIR, 256)):
            bm = C.c_int()
            assert lib.bmb_gemm_schedule_check(bmb.MATH_TF32, flags, 1, M, N, K, 148, C.byref(bm), None, None, None) == 0
            assert bm.value == want


def test_checkpoint_header_reads_the_gpt1_layout(bmb, tmp_path):
    """bmb_checkpoint_header on a file laid out by hand as src/train_gpt.cu:175-193 writes it (magic,
    GPTConfig, nvocab, vocabulary, parameters), without and with the appended optimiser section."""
    import struct
    import numpy as np
    cfg = (32, 5, 128, 1, 2, 8)                       # max_seq_len, vocab, padded vocab, layers, heads, width
    L, Cw, Vp, maxT = cfg[3], cfg[5], cfg[2], cfg[0]
    nparams = Vp * Cw + maxT * Cw + L * (2 * Cw + 3 * Cw * Cw + 3 * Cw + Cw * Cw + Cw + 2 * Cw + 4 * Cw * Cw + 4 * Cw + 4 * Cw * Cw + Cw) + 2 * Cw
    itos = b"\nabcd"
    params = np.arange(nparams, dtype=np.float32)
    plain, full = tmp_path / "plain.bin", tmp_path / "full.bin"
    head = struct.pack("<i6ii", 0x47505431, *cfg, len(itos)) + itos
    plain.write_bytes(head + params.tobytes())
    full.write_bytes(head + params.tobytes() + struct.pack("<2i", 0x4F424D42, 77) + params.tobytes() * 2)
    lib = bmb.lib()
    for path, want_opt, want_step in ((plain, 0, 0), (full, 1, 77)):
        hc, nv, opt, step = bmb.TrainConfig(), C.c_int(), C.c_int(-1), C.c_int(-1)
        buf = C.create_string_buffer(16)
        assert lib.bmb_checkpoint_header(str(path).encode(), C.byref(hc), C.byref(nv), buf, 16, C.byref(opt), C.byref(step)) == 0
        assert (hc.max_seq_len, hc.vocab_size, hc.padded_vocab, hc.n_layer, hc.n_head, hc.n_embd) == cfg
        assert nv.value == len(itos) and buf.raw[:len(itos)] == itos
        assert (opt.value, step.value) == (want_opt, want_step)
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"\0" * 64)
    assert lib.bmb_checkpoint_header(str(bad).encode(), None, None, None, 0, None, None) != 0
    assert b"not a GPT1 checkpoint" in lib.bmb_last_error()


def test_registry_csv_feeds_the_reference_merge_tool(tmp_path):
    """kernel_bench.py's CSV writer, given made-up numbers, produces files the reference's
    tools/merge_runs.py merges (it keys on kernel_id, kernel, size and reads the four float columns)."""
    import importlib.util
    import json
    import sys
    spec = importlib.util.spec_from_file_location("kernel_bench", os.path.join(ROOT, "bare-metal-bard_b200", "kernel_bench.py"))
    kb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(kb)
    runs = []
    for i in range(3):
        p = tmp_path / ("run%d.csv" % i)
        rows = [dict(kernel_id=k, kernel=n, size=s, gflops_best=1000.0 * k + s + i, gflops_median=900.0 * k + s,
                     cublas_gflops_best=50000.0, pct_of_cublas=(1000.0 * k + s + i) / 500.0)
                for k, n in ((1, "simt_fp32"), (2, "tcgen05_tf32")) for s in (1024, 2048)]
        kb.append_csv(str(p), rows[:2])
        kb.append_csv(str(p), rows[2:])          # appending must not repeat the header
        runs.append(str(p))
    text = open(runs[0]).read().splitlines()
    assert text[0] == "kernel_id,kernel,size,gflops_best,gflops_median,cublas_gflops_best,pct_of_cublas" and len(text) == 5
    assert text[1] == "1,simt_fp32,1024,2024.00,1924.00,50000.00,4.05"
    try:
        ref = json.load(open(os.path.join(ROOT, "BASELINE.json"))).get("reference_path")
    except Exception:
        ref = None
    tool = os.path.join(ref or "", "tools", "merge_runs.py")
    if not (ref and os.path.exists(tool)):
        pytest.skip("reference checkout absent: merge_runs.py not run")
    out = tmp_path / "merged.csv"
    r = subprocess.run([sys.executable, tool, str(out)] + runs, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    merged = out.read_text().splitlines()
    assert merged[0] == text[0] and len(merged) == 5 and merged[1].startswith("1,simt_fp32,1024,2025.00")


@pytest.mark.parametrize("L,E,V,maxT", [(12, 768, 50304, 1024), (1, 32, 96, 16), (2, 64, 128, 32), (3, 32, 96, 16), (5, 64, 256, 64)])
def test_step_plan_chunks_partition_the_parameters_and_pieces_cover_the_step(bmb, L, E, V, maxT):
    """The overlapped exchange's plans (host logic, no GPU; 1 = reduces under backward, 2 = also updates under the
    next forward): the three chunks are disjoint ranges that
    together cover every parameter exactly once and hold the layers they are named for; the pieces run
    every unit once, in order; a chunk's update is awaited by the first piece that reads its layers and
    its reduce follows the piece that writes the last of its gradients."""
    import numpy as np
    cfg = bmb.TrainConfig(maxT, V, V, L, 2, E, 2, maxT, 1, 1, 1, 0.9, 0.95, 1e-8, 0.0, 1.0)
    ranges = (C_ull * (3 * 16 * 2))()
    nranges, pieces, npieces = (C.c_int * 3)(), (C.c_int * 20)(), C.c_int(0)
    lib = bmb.lib()
    total = V * E + maxT * E + L * (2 * E + 3 * E * E + 3 * E + E * E + E + 2 * E + 4 * E * E + 4 * E + 4 * E * E + E) + 2 * E
    for overlapped in (0, 1, 2):
        assert lib.bmb_trainer_step_plan(C.byref(cfg), overlapped, ranges, nranges, pieces, C.byref(npieces)) == 0
        cover = np.zeros(total, dtype=np.int8)
        owner = np.full(total, -1, dtype=np.int8)
        for k in range(3):
            for q in range(nranges[k]):
                off, ln = ranges[(k * 16 + q) * 2], ranges[(k * 16 + q) * 2 + 1]
                assert off % 4 == 0 and ln % 4 == 0 and ln > 0 and off + ln <= total
                cover[off:off + ln] += 1
                owner[off:off + ln] = k
        assert cover.min() == 1 and cover.max() == 1
        ps = [tuple(pieces[4 * i:4 * i + 4]) for i in range(npieces.value)]
        U = 2 * L + 4
        assert ps[0][0] == 0 and ps[-1][1] == U and all(a[1] == b[0] for a, b in zip(ps, ps[1:]))
        if not overlapped or L < 2:
            assert len(ps) == 1 and nranges[0] == 1 and ranges[0] == 0 and ranges[1] == total
            continue
        # the chunk every layer's first tensor (ln1w, right after wte and wpe) lives in
        ln1w = V * E + maxT * E
        layer_chunk = [int(owner[ln1w + l * E]) for l in range(L)]
        assert layer_chunk[0] == 0 and layer_chunk == sorted(layer_chunk)
        assert owner[0] == 0 and owner[V * E] == 0 and owner[total - 1] == 2          # embeddings in A, final layernorm in C
        first_use, last_write = {}, {}
        for i, (u0, u1, needs, reduces) in enumerate(ps):
            for u in range(u0, u1):
                if u == 0 or u == L + 1: ks = [0]                       # embedding; head (tied weights)
                elif 1 <= u <= L: ks = [layer_chunk[u - 1]] + ([2] if u == L else [])   # the last layer also applies the final layernorm
                elif u == L + 2: ks = [0, 2, layer_chunk[L - 1]]      # head backward: dwte, final layernorm, last layer's second bias
                elif u <= 2 * L + 2:
                    l = 2 * L + 2 - u
                    ks = [layer_chunk[l]] + ([layer_chunk[l - 1]] if l > 0 else [])
                else: ks = [0]
                for k in ks:
                    first_use.setdefault(k, i)
                    if u >= L + 2: last_write[k] = i
        for k in (0, 1, 2):
            if nranges[k] == 0:
                continue
            # (mode 1: only the reduces are overlapped; the first piece waits for the last chunk's update, which the
            #  exchange stream finishes after all the others)
            waits = [i for i, pc in enumerate(ps) if pc[2] == k or (overlapped == 1 and pc[2] == 2)]
            reds = [i for i, pc in enumerate(ps) if pc[3] == k]
            assert waits and waits[0] <= first_use[k], (k, ps)
            assert len(reds) == 1 and reds[0] >= last_write[k], (k, ps)
