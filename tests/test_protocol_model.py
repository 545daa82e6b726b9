"""The mbarrier protocol of the key-loop tcgen05 kernels, checked on the CPU with a discrete-event model
(tests/protocol_model.py): random latencies, random piece shapes, hardware parity semantics, ownership assertions on
every tensor-memory buffer and ring stage.  No GPU run can show the absence of a race; a few hundred random schedules of
the model at least show the protocol has none that depends on who is faster."""
import random

import pytest

from protocol_model import forward_kernel, key_major_kernel, outcome, query_major_kernel, single_shot_backward_kernel

RUNS = 250


def _pieces(seed):
    rng = random.Random(seed)
    return [rng.randint(1, 25) for _ in range(rng.randint(1, 4))]          # odd and even unit lengths, units of one job


def test_key_major_kernel_protocol_has_no_hazard_or_deadlock():
    """attn_dkv_pooled_loop_tc_kernel as built: one S^T / dP^T thread, one dV / dK thread, three buffers, barriers per buffer."""
    for seed in range(RUNS):
        assert outcome(key_major_kernel, seed, _pieces(seed)) == "ok", seed


def test_query_major_kernel_protocol_has_no_hazard_or_deadlock():
    """attn_dq_pooled_loop_tc_kernel as built: one S / dP thread, one dQ thread."""
    for seed in range(RUNS):
        rng = random.Random(seed)
        assert outcome(query_major_kernel, seed, rng.randint(1, 7), rng.choice([4, 6, 18])) == "ok", seed


@pytest.mark.parametrize("passes", [1, 2])
def test_forward_kernel_protocol_has_no_hazard_or_deadlock(passes):
    """attn_fwd_pooled_loop_tc_kernel as built, in its one-pass form (odd and even chunk counts: with 9 chunks the groups
    swap the parity of their first job from tile to tile) and in the two-pass form that redoes marked rows."""
    for seed in range(RUNS):
        rng = random.Random(seed)
        assert outcome(forward_kernel, seed, rng.randint(1, 6), rng.choice([2, 3, 8, 9]), passes) == "ok", seed


def test_model_catches_the_parity_hazard_of_two_score_threads():
    """The model has teeth: S / dP of even and odd jobs on TWO threads with barriers per BUFFER is the variant that read
    scores before they were written on the GPU.  A softmax group asks for the second completion of a barrier whose first
    completion belongs to the other thread and has not happened yet; the parity test passes.  The model finds it within
    a few schedules, in both kernels."""
    bad_kv = sum(outcome(key_major_kernel, s, _pieces(s), score_threads=2) != "ok" for s in range(60))
    bad_q = sum(outcome(query_major_kernel, s, 4, 6, score_threads=2) != "ok" for s in range(60))
    assert bad_kv > 0 and bad_q > 0


@pytest.mark.parametrize("kernel", ["key_major", "query_major"])
def test_barriers_per_job_number_mod_6_make_two_score_threads_safe(kernel):
    """With sdp_ready / buf_free indexed by the job number mod 6 every barrier has one committing thread and one waiting
    thread or group that meet its phases in order: the two-thread variant is then safe (it ran parity-green with device
    checks on, and no faster than the one-thread form, which is why the kernels keep the simpler one)."""
    for seed in range(RUNS):
        if kernel == "key_major":
            r = outcome(key_major_kernel, seed, _pieces(seed), score_threads=2, score_barriers=6)
        else:
            rng = random.Random(seed)
            r = outcome(query_major_kernel, seed, rng.randint(1, 7), rng.choice([4, 6, 18]), score_threads=2, score_barriers=6)
        assert r == "ok", seed


def _single_shot_case(seed):
    rng = random.Random(seed)
    return rng.randint(0, 9), rng.randint(1, 14), rng.choice([2, 4, 8, 128])       # first tile, tiles of the CTA, tiles per head


def test_single_shot_backward_protocol_has_no_hazard_or_deadlock():
    """attn_bwd_pooled_tc_kernel as built: TMA producer, two MMA-issuing threads (S / dP / dQ; the transposed products) that
    both commit out_ready and mma_done, twelve softmax warps, four drain warps; CTA ranges that start on odd tiles, cross
    parents and heads, and end in the middle of a parent."""
    for seed in range(RUNS):
        assert outcome(single_shot_backward_kernel, seed, *_single_shot_case(seed)) == "ok", seed


def test_model_catches_a_stage_freed_by_one_issuer_only_and_an_unguarded_overwrite():
    """Two mutations of that protocol the model must catch: mma_done counting only one thread's commit (the producer then
    reloads Q / dO under the other thread's products) and softmax warps that do not wait for the previous tile's
    products before they overwrite P / dS."""
    one = sum(outcome(single_shot_backward_kernel, s, *_single_shot_case(s), mma_done_count=1) != "ok" for s in range(80))
    two = sum(outcome(single_shot_backward_kernel, s, *_single_shot_case(s), softmax_waits_for_products=False) != "ok" for s in range(80))
    assert one > 0 and two > 0
