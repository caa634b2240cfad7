"""The CPU oracle (oracle/sampler_oracle.c) against the fixtures that pin it:
tokens produced by the reference's own unmodified sampler.cpp (tests/golden), the
known-answer argmax cases of the reference's own tests, and known-answer coins."""
import hashlib

import numpy as np
import pytest

import oracle
from executorch_b200 import workloads as W


def test_xorshift_known_answers(restatement):
    # states and coins of xorshift64* as specified in sampler.cpp:210-220
    coins, states = restatement.coins(1, 3)
    assert states == [33554433, 1126174793148417, 3659449627584515]
    assert np.allclose(coins, [0.280835032, 0.671137214, 0.725846112], atol=0, rtol=1e-7)
    assert restatement.coins(0, 3)[0] == [0.0, 0.0, 0.0]  # zero is a fixed point
    assert np.allclose(restatement.coins(42, 3)[0], [0.339085221, 0.782255828, 0.790136993], rtol=1e-7)
    assert np.allclose(restatement.coins(2, 3)[0], [0.561670065, 0.342274487, 0.462054551], rtol=1e-7)


def test_reference_argmax_fixtures(restatement):
    # extension/llm/sampler/test/test_sampler.cpp:19-43: uniform [0,1) logits with
    # element 396 set to 1.0, temperature 0 -> 396, for float and for half
    g = np.random.default_rng(7)
    x = g.random((1, 32000), dtype=np.float32) * np.float32(0.999)
    x[0, 396] = 1.0
    seeds = np.zeros(1, dtype=np.uint64)
    assert restatement.sample_rows(x, 0.0, 0.9, seeds)[0] == 396
    xh = x.astype(np.float16)
    xh[0, 396] = 1.0
    xh[xh >= 1.0] = np.float16(0.999)
    xh[0, 396] = 1.0
    assert restatement.sample_rows(xh.view(np.uint16), 0.0, 0.9, seeds, dtype="fp16")[0] == 396
    # extension/llm/runner/test/test_text_decoder_runner.cpp:83-140: {0.1,0.2,0.8,0.4} -> 2
    small = np.array([[0.1, 0.2, 0.8, 0.4]], dtype=np.float32)
    assert restatement.sample_rows(small, 0.0, 0.9, seeds)[0] == 2
    assert restatement.sample_rows(W.f32_to_bf16_bits(small), 0.0, 0.9, seeds, dtype="bf16")[0] == 2
    assert restatement.sample_rows(small.astype(np.float16).view(np.uint16), 0.0, 0.9, seeds, dtype="fp16")[0] == 2
    # extension/llm/runner/test/test_text_llm_runner.cpp:656-715: argmax 3, masked -> 2, -> 1
    lg = np.array([[0.1, 0.2, 0.3, 0.4]], dtype=np.float32)
    assert restatement.sample_rows(lg, 0.0, 0.9, seeds)[0] == 3
    lg[0, 3] = -np.inf
    assert restatement.sample_rows(lg, 0.0, 0.9, seeds)[0] == 2
    lg[0, 2] = -np.inf
    assert restatement.sample_rows(lg, 0.0, 0.9, seeds)[0] == 1


def test_argmax_edge_semantics(restatement):
    seeds = np.zeros(1, dtype=np.uint64)
    ties = np.array([[1.0, 3.0, 3.0, 2.0, 3.0]], dtype=np.float32)
    assert restatement.sample_rows(ties, 0.0, 0.9, seeds)[0] == 1  # lowest index wins
    zeros = np.array([[-0.0, 0.0, -1.0]], dtype=np.float32)
    assert restatement.sample_rows(zeros, 0.0, 0.9, seeds)[0] == 0  # -0 == +0
    nan0 = np.array([[np.nan, 5.0, 7.0]], dtype=np.float32)
    assert restatement.sample_rows(nan0, 0.0, 0.9, seeds)[0] == 0  # NaN at 0 is never replaced
    nan1 = np.array([[1.0, np.nan, 0.5]], dtype=np.float32)
    assert restatement.sample_rows(nan1, 0.0, 0.9, seeds)[0] == 0  # NaN never wins
    u16 = np.array([[5, 65535, 7, 65535]], dtype=np.uint16)
    assert restatement.sample_rows(u16, 0.0, 0.9, seeds, dtype="u16")[0] == 1


def test_small_cases_match_reference_tokens(restatement, golden):
    z, meta = golden
    n = 0
    for m in meta:
        if m["kind"] != "small":
            continue
        x, seeds = z[m["key"] + "_x"], z[m["key"] + "_seeds"]
        for si, (t, p) in enumerate(m["settings"]):
            got = restatement.sample_rows(x, t, p, seeds, dtype=m["dtype"])
            want = z[f"{m['key']}_st{si}"]
            assert np.array_equal(got, want), (m, t, p)
            n += len(want)
            if m["dtype"] == "fp32" or t == 0.0 or not (0.0 < p < 1.0):
                # no equal probabilities to reorder: the shipped std::sort build agrees too
                assert np.array_equal(got, z[f"{m['key']}_sh{si}"]), (m, t, p)
    assert n >= 1000


def test_workload_cases_match_reference_tokens(restatement, golden):
    z, meta = golden
    for m in meta:
        if m["kind"] != "workload":
            continue
        cfg = W.CONFIGS[m["name"]]
        x = W.rows_numpy(m["name"], m["row_ids"])
        assert hashlib.sha256(x.tobytes()).hexdigest() == m["sha256"], "input generator drifted"
        seeds = np.asarray(m["row_ids"], dtype=np.uint64)
        for si, (t, p) in enumerate(m["settings"]):
            got = restatement.sample_rows(x, t, p, seeds, dtype=cfg.dtype, threads=4)
            assert np.array_equal(got, z[f"w_{m['name']}_st{si}"]), (m["name"], t, p)


def test_topk_matches_reference_tokens(restatement, golden):
    z, meta = golden
    for m in meta:
        if m["kind"] != "topk":
            continue
        x, seeds = z[m["key"] + "_x"], z[m["key"] + "_seeds"]
        for k in m["ks"]:
            got = restatement.sample_rows(x, m["temperature"], m["topp"], seeds, topk=k)
            assert np.array_equal(got, z[f"{m['key']}_k{k}"]), (m["vocab"], k)
    x = W.rows_numpy("c1", list(range(100)))
    got = restatement.sample_rows(x, 0.8, 0.9, np.arange(100, dtype=np.uint64), topk=40)
    assert np.array_equal(got, z["k_c1_k40"])


def test_decode_loop_sequence(restatement, golden):
    z, _ = golden
    row = W.bf16_bits_to_f32(z["seq_x"])
    got = restatement.sample_sequence(row, 0.7, 0.9, 12345, 64)
    assert np.array_equal(got, z["seq_tok"])


def test_rng_advances_once_per_sampled_row_only(restatement):
    x = W.rows_numpy("c1", [0, 1, 2], vocab=512)
    seeds = np.array([5, 6, 7], dtype=np.uint64)
    _, st = restatement.sample_rows(x, 0.0, 0.9, seeds, return_states=True)
    assert np.array_equal(st, seeds)  # greedy draws no coin (sampler.cpp:226-228)
    _, st = restatement.sample_rows(x, 0.8, 0.9, seeds, return_states=True)
    for s0, s1 in zip(seeds, st):
        assert restatement.coins(int(s0), 1)[1][0] == int(s1)


@pytest.mark.skipif(not oracle.Reference.available(True), reason="oracle/_ref not built here")
def test_restatement_equals_compiled_reference_live(restatement):
    """Where the compiled reference is present, re-check agreement on fresh inputs."""
    ref = oracle.Reference(stable=True)
    for name, ids, vocab in (("c1", range(300, 340), None), ("c3", range(40, 48), None),
                             ("c4", [5, 2050], 20000), ("c5", range(20, 24), None)):
        cfg = W.CONFIGS[name]
        x = W.rows_numpy(name, list(ids), vocab=vocab)
        seeds = np.asarray(list(ids), dtype=np.uint64) + 99
        for t, p in ((0.0, 0.9), (cfg.temperature, 1.0), (cfg.temperature, cfg.topp), (0.5, 0.3)):
            a = restatement.sample_rows(x, t, p, seeds, dtype=cfg.dtype, threads=4)
            b = ref.sample_rows(x, t, p, seeds, dtype=cfg.dtype, threads=4)
            assert np.array_equal(a, b), (name, t, p)
