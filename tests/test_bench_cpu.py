"""Host-side checks of bench.py: the algorithmic work figures and the command line contract."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_work_of_the_named_configs():
    b = _bench()
    # config 4 (chunk-visible, T = 65536, Hq = 32, D = 128, L = 32): forward 35.48, backward 88.69,
    # together 124.17 TFLOP; sequence-only twin 123.15 TFLOP
    mode, B, T, Hkv, G, D, L = b.WORKLOADS[b.DEFAULT_WORKLOAD]
    fwd = b.flops(mode, B, T, Hkv, G, D, L, fwd=True, bwd=False)
    both = b.flops(mode, B, T, Hkv, G, D, L, fwd=True, bwd=True)
    assert abs(fwd / 1e12 - 35.48) < 0.01
    assert abs(both / 1e12 - 124.17) < 0.01
    twin = b.flops(*b.WORKLOADS["config4_seq_only_twin_T65536"], fwd=True, bwd=True)
    assert abs(twin / 1e12 - 123.15) < 0.01
    # config 2 forward 0.1391 TFLOP; config 3 forward + backward 0.060 TFLOP; config 5 0.056 TFLOP
    assert abs(b.flops(*b.WORKLOADS["config2_causal_T4096"], fwd=True, bwd=False) / 1e12 - 0.1391) < 1e-3
    assert abs(b.flops(*b.WORKLOADS["config3_fda_T8192"], fwd=True, bwd=True) / 1e12 - 0.060) < 1e-3
    assert abs(b.flops(*b.WORKLOADS["config5_deit_noncausal_T197"], fwd=True, bwd=True) / 1e12 - 0.056) < 1e-3


def test_chunk_visible_pairs_match_a_direct_count():
    b = _bench()
    T, G, L, C = 100, 4, 3, 64
    cb = C // G
    direct = 0
    for t in range(T):
        direct += (t + 1) + (t - (t // cb) * cb + 1) * L     # sequence keys + depth rows of the chunk so far
    assert b.pairs("chunk", 1, T, 1, G, L) == direct * G


def test_reference_arm_prints_one_json_line_and_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == ""
    env = dict(os.environ, RANK="0", WORLD_SIZE="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-sample-T", "512"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0


def test_triton_baseline_arm_reports_unavailable_without_a_gpu():
    """The reference-Triton leg never raises: without a CUDA device (or without the reference
    install) it prints one JSON line that says why it has no numbers."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "triton_baseline"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "triton_baseline"
    import torch
    if not torch.cuda.is_available():
        assert "unavailable" in line and line["results"] == []


def test_kernel_attribution_tables_cover_the_same_kernels():
    b = _bench()
    assert set(b.OWNED_MATMULS) == set(b.EXECUTED_MATMULS)
    # the forward owns both of its matmuls; a two-kernel backward owns three of the five algorithmic ones
    assert b.OWNED_MATMULS["tc_fwd"] == 2 and b.OWNED_MATMULS["tc_dq"] + b.OWNED_MATMULS["tc_dkv"] == 3
    for name in b.OTHER_WORKLOADS:
        assert name in b.WORKLOADS
    # the published shape: 14 * d * Hq * (T (T + 1) / 2 + T L) FLOP
    fl = b.flops(*b.WORKLOADS["published_causal_T65536_d64"], fwd=True, bwd=True)
    assert abs(fl - 14 * 64 * 64 * (65536 * 65537 // 2 + 65536 * 64)) < 1


def test_tensor_pipe_model_counts():
    """The block and instruction counts behind roofline.tensor_pipe: config 4 executes one 128 x 128
    block per (query tile, visible key tile) and eight depth blocks per query tile; the forward
    issues 8 + 8 matmul instructions per block at D = 128, the backward kernels 32 score
    instructions plus 8 (dq) or 16 (dk/dv) update instructions."""
    b = _bench()
    mode, B, T, Hkv, G, D, L = b.WORKLOADS["config4_chunk_visible_T65536"]
    seq, dep = b.executed_blocks(mode, B, T, Hkv, G, L)
    n_qt = T * G // 128
    assert dep == B * Hkv * n_qt * 8
    # query tile i covers positions 32 i .. 32 i + 31 and sees ceil((32 i + 32) / 128) key tiles
    assert seq == B * Hkv * sum(-(-(32 * i + 32) // 128) for i in range(n_qt))
    # at least the algorithmic pairs, at most one extra (diagonal) tile per query tile
    alg = b.pairs(mode, B, T, Hkv, G, 0) / (128 * 128)
    assert alg <= seq <= alg + B * Hkv * n_qt
    assert b.mma_mix("tc_fwd", 128) == {"ss_n128": 8, "ts_n128": 8}
    assert b.mma_mix("tc_dq", 128) == {"ts_n64": 32, "ss_n128": 8}
    assert b.mma_mix("tc_dkv", 128) == {"ts_n64": 32, "ss_n128": 16}
    assert b.mma_mix("tc_fwd", 64) == {"ss_n128": 4, "ts_n64": 8}
    assert b.mma_mix("fda_fwd", 128) is None
    # bytes through the shared-memory port per 128 x 128 block
    assert sum(b.smem_bytes("tc_fwd", 128).values()) == 131072
    assert sum(b.smem_bytes("tc_dq", 128).values()) == 229376
    assert sum(b.smem_bytes("tc_dkv", 128).values()) == 328704
    assert sum(b.smem_bytes("tc_fwd", 64).values()) == 65536
    assert b.mma_mix("tc_dkv", 64) == {"ts_n64": 32} and b.mma_mix("tc_dq", 64) == {"ts_n64": 24}
    assert b.smem_bytes("tc_dq", 64) == {"mma_operands": 49152, "tma_fill": 32768, "softmax_stores": 0}
    assert b.smem_bytes("fda_fwd", 128) is None
