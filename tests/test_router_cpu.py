"""The routing session of the native runtime as the Python layer uses it (no GPU: the router is host code). One
line of the policy file changes what the trainer's communicators do."""
import torch

from coccl_b200.parallel.comm import ALGO_AR_ONESHOT, ALGO_AR_TWOSHOT, NATIVE, Policy, Router


def _decide(policy, role, op, dtype, count, n=2, explicit=-1):
    r = Router.of(policy, n)
    return r, r.decide(role, op, dtype, count, n, 0, explicit)


def test_training_policy_routes_roles():
    pol = Policy()   # the shipped training policy
    r, d = _decide(pol, 1, "reduce_scatter", torch.float32, 1 << 24)
    assert r.training_mode() and d.compressed and d.fusable and d.compressor == b"sdp4bit"
    assert (d.codec.bits, d.codec.group, d.codec.hadamard) == (4, 128, 1)
    _, d = _decide(pol, 1, "all_gather", torch.bfloat16, 1 << 24)
    assert d.compressed and d.fusable and d.delta and (d.codec.bits, d.codec.group) == (8, 2048)   # subAdd: parameter deltas
    _, d = _decide(pol, 2, "all_gather", torch.bfloat16, 1 << 22)
    assert d.compressed and d.compressor == b"fp8block" and d.codec.kind == 1
    _, d = _decide(pol, 2, "reduce_scatter", torch.bfloat16, 1 << 23)
    assert d.compressed and d.compressor == b"fp8block"
    # below the threshold, unknown role, pipeline traffic, no policy slot: native
    assert not _decide(pol, 1, "reduce_scatter", torch.float32, 1000)[1].compressed
    assert not _decide(pol, 0, "reduce_scatter", torch.float32, 1 << 24)[1].compressed
    assert not _decide(pol, 3, "sendrecv", torch.bfloat16, 1 << 24)[1].compressed
    assert not _decide(pol, 1, "all_reduce", torch.float32, 1 << 24)[1].compressed
    assert Router.of(NATIVE, 2) is None


def test_one_line_of_the_policy_file_changes_the_decision():
    base = Policy.training(threshold_bytes=0)
    r0, d0 = _decide(base, 1, "reduce_scatter", torch.float32, 1 << 20)
    edited = Policy(toml=base.toml.replace("quantBits = 4", "quantBits = 8"))
    r1, d1 = _decide(edited, 1, "reduce_scatter", torch.float32, 1 << 20)
    assert d0.codec.bits == 4 and d1.codec.bits == 8
    assert r0.config_hash() != r1.config_hash()
    assert "quantBits = 8" in r1.effective_config() or "quantBits=8" in r1.effective_config()
    # threshold: `bytes <= threshold` stays native, bytes scaled by the ranks for a reduce-scatter
    thr = Policy.training(threshold_bytes=(1 << 20) * 4 * 2)
    assert not _decide(thr, 1, "reduce_scatter", torch.float32, 1 << 20)[1].compressed
    assert _decide(thr, 1, "reduce_scatter", torch.float32, (1 << 20) + 2)[1].compressed
    # a rejected file is an error, not a silent native run
    try:
        Router.of(Policy(toml=base.toml.replace('mode = "training"', 'mode = "nonsense"')), 2)
    except RuntimeError as e:
        assert "mode" in str(e)
    else:
        raise AssertionError("bad policy accepted")


def test_selector_follows_measurements_unless_forced():
    pol = Policy.normal("sdp4bit", threshold_bytes=0, autotune=True)
    r, d = _decide(pol, 0, "all_reduce", torch.float32, 1 << 18)
    assert d.compressed and d.algorithm == ALGO_AR_TWOSHOT          # no measurements: the heuristic prefers two-shot
    # timings as the framework layer feeds them: one-shot wins at 1 MiB, two-shot at 64 MiB
    r.set_measured("all_reduce", torch.float32, 2, 20, ALGO_AR_ONESHOT, 10e-6)
    r.set_measured("all_reduce", torch.float32, 2, 20, ALGO_AR_TWOSHOT, 14e-6)
    r.set_measured("all_reduce", torch.float32, 2, 26, ALGO_AR_ONESHOT, 900e-6)
    r.set_measured("all_reduce", torch.float32, 2, 26, ALGO_AR_TWOSHOT, 300e-6)
    assert r.decide(0, "all_reduce", torch.float32, 1 << 18, 2, 0).algorithm == ALGO_AR_ONESHOT    # 1 MiB bucket
    assert r.decide(0, "all_reduce", torch.float32, 1 << 19, 2, 0).algorithm == ALGO_AR_ONESHOT    # 2 MiB: nearest below
    assert r.decide(0, "all_reduce", torch.float32, 1 << 24, 2, 0).algorithm == ALGO_AR_TWOSHOT    # 64 MiB
    assert r.decide(0, "all_reduce", torch.float32, 1 << 12, 2, 0).algorithm == ALGO_AR_ONESHOT    # below all: nearest above
    forced = Policy.normal("sdp4bit", threshold_bytes=0, autotune=True, all_reduce_algorithm="twoshot")
    rf, _ = _decide(forced, 0, "all_reduce", torch.float32, 1 << 18)
    rf.set_measured("all_reduce", torch.float32, 2, 20, ALGO_AR_ONESHOT, 1e-6)
    rf.set_measured("all_reduce", torch.float32, 2, 20, ALGO_AR_TWOSHOT, 9e-6)
    assert rf.decide(0, "all_reduce", torch.float32, 1 << 18, 2, 0).algorithm == ALGO_AR_TWOSHOT   # the file wins
    # uncompressed all-reduce: NCCL or the multimem kernel, from measurements
    big = Policy.normal("sdp4bit", threshold_bytes=1 << 30, autotune=True)
    rb, d = _decide(big, 0, "all_reduce", torch.float32, 1 << 18)
    assert not d.compressed and d.native_variant == 0
    rb.set_measured_native(torch.float32, 2, 20, 0, 30e-6)
    rb.set_measured_native(torch.float32, 2, 20, 1, 12e-6)
    assert rb.decide(0, "all_reduce", torch.float32, 1 << 18, 2, 0).native_variant == 1


def test_explicit_call_ignores_the_threshold_and_codecs_without_tile_form_are_reported():
    pol = Policy.normal("sdp4bit", threshold_bytes=1 << 30)
    assert not _decide(pol, 0, "all_reduce", torch.float32, 1 << 18)[1].compressed
    d = _decide(pol, 0, "all_reduce", torch.float32, 1 << 18, explicit=ALGO_AR_ONESHOT)[1]
    assert d.compressed and d.algorithm == ALGO_AR_ONESHOT
    ans = Policy.normal("ans", {"probBits": 10}, threshold_bytes=0)
    d = _decide(ans, 0, "all_gather", torch.float32, 1 << 20)[1]
    assert d.compressed and not d.fusable and d.compressor == b"ans"     # served by the staged pipeline of the C API
    zfp = Policy.normal("zfp", {"rate": 8}, threshold_bytes=0)
    d = _decide(zfp, 0, "all_gather", torch.bfloat16, 1 << 20)[1]
    assert d.compressed and d.fusable and d.codec.kind == 4 and d.codec.bits == 8
    taco = Policy.normal("taco", {"groupSize": 256}, threshold_bytes=0)
    d = _decide(taco, 0, "all_to_all", torch.float32, 1 << 20)[1]
    assert d.compressed and d.fusable and d.codec.kind == 3 and d.codec.group == 256
    # integer payloads: a lossy codec leaves them native, a bytewise-lossless one takes them
    assert not _decide(zfp, 0, "all_gather", torch.int32, 1 << 20)[1].compressed
    assert _decide(ans, 0, "all_gather", torch.int32, 1 << 20)[1].compressed


def test_policy_file_limits_the_ctas_of_the_fused_kernels():
    """[runtime] fused_kernel_max_ctas: the share of the GPU a fused kernel may take (its CTAs wait on one another, so
    whatever runs next to it must leave them resident); the communicator launches with that limit."""
    base = Policy.training(threshold_bytes=0)
    assert Router.of(base, 2).fused_max_ctas() == 0
    assert "fused_kernel_max_ctas = 0" in base.toml
    limited = Policy(toml=base.toml.replace("fused_kernel_max_ctas = 0", "fused_kernel_max_ctas = 96", 1))
    r = Router.of(limited, 2)
    assert r.fused_max_ctas() == 96 and "fused_kernel_max_ctas = 96" in r.effective_config()
    import pytest
    bad = Policy(toml=base.toml.replace("fused_kernel_max_ctas = 0", "fused_kernel_max_ctas = -3", 1))
    with pytest.raises(Exception):
        Router.of(bad, 2)
