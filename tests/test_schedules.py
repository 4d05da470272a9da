"""Schedule generators against instruction streams recorded from the reference implementation
(its pure-Python schedule classes executed in isolation), plus structural invariants."""
import itertools

import pytest

from merak_b200.pipeline import schedules as S

GOLDEN = {
    ("1f1b", 2, 4): [
        "L0+F0 | SA0 | L1+F1 | SARG1>0+B0 | L2+F2 | SARG2>1+B1 | L0+F0 | SARG0>2+B2 | RG0+B0+RT+RD+OPT",
        "RA0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SGRA1>0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1+RT+RD+OPT",
    ],
    ("ds_default", 2, 4): [
        "L0+F0 | SA0 | L1+F1 | SA1+RG0+B0 | L2+F2 | SA2+RG1+B1 | L0+F0 | SA0+RG2+B2 | RG0+B0+RT+RD+OPT",
        "RA0+L0+F0 | B0 | RA1+SG0+L1+F1 | B1 | RA0+SG1+L0+F0 | B0 | RA1+SG0+L1+F1 | B1 | SG1+RT+RD+OPT",
    ],
    ("1f1b", 4, 4): [
        "L0+F0 | SA0 | L1+F1 | SA1 | L2+F2 | SA2 | L3+F3 | SARG3>0+B0 | RG1+B1 | RG2+B2 | RG3+B3+RT+RD+OPT",
        "RA0+F0 | SA0 | RA1+F1 | SA1 | RA2+F2 | SARG2>0+B0 | SGRA0>3+F3 | SARG3>1+B1 | SG1 | RG2+B2 | SG2 | RG3+B3 | SG3+RT+RD+OPT",
        "RA0+F0 | SA0 | RA1+F1 | SARG1>0+B0 | SGRA0>2+F2 | SARG2>1+B1 | SGRA1>0+F0 | SARG0>2+B2 | SG2 | RG0+B0 | SG0 | RT+RD+OPT",
        "RA0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SGRA1>0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1 | RT+RD+OPT",
    ],
    ("pre_recompute_1f1b", 4, 4): [
        "L0+F0 | SA0 | L1+PF1 | SA1 | L2+PF2 | SA2 | L3+PF3 | SARG3>0+B0 | RRG1+B1 | RRG2+B2 | RRG3+B3+RS+RT+RD+OPT",
        "RA0+F0 | SA0 | RA1+F1 | SA1 | RA2+PF2 | SARG2>0+B0 | SGRA0>3+PF3 | SARG3>1+B1 | SG1 | RRG2+B2 | SG2 | RRG3+B3 | SG3+RS+RT+RD+OPT",
        "RA0+F0 | SA0 | RA1+F1 | SARG1>0+B0 | SGRA0>2+F2 | SARG2>1+B1 | SGRA1>0+PF0 | SARG0>2+B2 | SG2 | RRG0+B0 | SG0 | RS+RT+RD+OPT",
        "RA0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SGRA1>0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1 | RT+RD+OPT",
    ],
    ("full_critical_path_1f1b", 4, 4): [
        "L0+F0 | SA0 | L1+PF1 | SA1 | L2+PF2 | SA2 | L3+PF3 | SARG3>0+B0 | RRG1+B1 | RRG2+B2 | RRG3+B3+RS+RT+RD+OPT",
        "RA0+PF0+RS | SA0 | RA1+F1 | SA1 | RA2+PF2 | SA2+RRG0+RS+B0 | SGRA0>3+PF3 | SARG3>1+B1 | SG1 | RRG2+B2 | SG2 | RRG3+B3 | SG3+RS+RT+RD+OPT",
        "RA0+PF0+RS | SA0 | RA1+PF1+RS | RA2+F2 | RRG0+SA1+RS+B0 | SG0+RRG1+SA2+RS+B1 | SGRA1>0+F0 | SARG0>2+B2 | SG2 | RG0+B0 | SG0 | RS+RT+RD+OPT",
        "RA0+L0+F0 | B0 | SG0+RA1+L1+F1 | B1 | SG1+RA0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1 | RT+RD+OPT",
    ],
    ("full_critical_path_1f1b", 2, 4): [
        "L0+PF0+RS | SA0 | L1+PF1+RS | RA2+L2+F2 | RRG0+SA1+RS+B0 | SG0+RRG1+SA2+RS+B1 | L0+F0 | SARG0>2+B2 | RG0+B0+RS+RT+RD+OPT",
        "RA0+L0+F0 | B0 | SG0+RA1+L1+F1 | B1 | SG1+RA0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1+RT+RD+OPT",
    ],
    ("full_critical_path_1f1b", 3, 6): [
        "L0+PF0+RS | SA0 | L1+F1 | SA1 | L2+F2 | SA2+RRG0+RS+B0 | L3+F3 | SARG3>1+B1 | L0+PF0 | SARG0>2+B2 | L1+PF1 | SARG1>3+B3 | RRG0+B0 | RRG1+B1+RS+RT+RD+OPT",
        "RA0+PF0+RS | SA0 | RA1+PF1+RS | RA2+F2 | RRG0+SA1+RS+B0 | SG0+RRG1+SA2+RS+B1 | SGRA1>0+F0 | SARG0>2+B2 | SGRA2>1+F1 | SARG1>0+B0 | SGRA0>2+F2 | SARG2>1+B1 | SG1 | RG2+B2 | SG2+RS+RT+RD+OPT",
        "RA0+L0+F0 | B0 | SG0+RA1+L1+F1 | B1 | SG1+RA0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SGRA1>0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1 | RT+RD+OPT",
    ],
}
GOLDEN_LAST_NO_RECOMPUTE_S2_S3 = [
    "RA0+PF0+RS | SA0 | RA1+F1 | RRG0+SA1+RS+B0 | SGRA0>2+F2 | SARG2>1+B1 | SGRA1>0+F0 | SARG0>2+B2 | SG2 | RG0+B0 | SG0 | RS+RT+RD+OPT",
    "RA0+L0+F0 | B0 | SG0+RA1+L1+F1 | B1 | SGRA1>0+L0+F0 | B0 | SGRA0>1+L1+F1 | B1 | SG1 | RT+RD+OPT",
]
NBUF = {("1f1b", 2, 4): [3, 2], ("1f1b", 4, 4): [4, 4, 3, 2], ("full_critical_path_1f1b", 3, 6): [4, 3, 2]}


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_golden_streams(key):
    name, stages, mbs = key
    for sid, want in enumerate(GOLDEN[key]):
        sched = S.make_schedule(name, mbs, stages, sid)
        assert S.format_steps(sched.steps()) == want, "%s stage %d" % (key, sid)
        if key in NBUF:
            assert sched.num_pipe_buffers() == NBUF[key][sid]


def test_last_no_recompute_golden():
    base = GOLDEN[("pre_recompute_1f1b", 4, 4)]
    for sid in range(4):
        got = S.format_steps(S.make_schedule("last_no_recompute_1f1b", 4, 4, sid).steps())
        want = base[sid] if sid < 2 else GOLDEN_LAST_NO_RECOMPUTE_S2_S3[sid - 2]
        assert got == want, sid


def test_inference_golden():
    want = ["L0+F0 | L1+SA0+F1 | L0+SA1+F0 | SA0", "L0+RA0+F0 | L1+RA1+F1 | L0+RA0+F0"]
    for sid in range(2):
        assert S.format_steps(S.InferenceSchedule(3, 2, sid).steps()) == want[sid]


def _simulate(name, stages, mbs):
    """Runs all stages in lock-step and checks that every send meets a matching receive in the
    same step (p2p calls are blocking pairs), that each micro-batch is forwarded and backwarded
    exactly once per stage, and that a backward never precedes its forward."""
    gens = [list(S.make_schedule(name, mbs, stages, s).steps()) for s in range(stages)]
    n = len(gens[0])
    assert all(len(g) == n for g in gens)
    fwd = [[] for _ in range(stages)]
    bwd = [[] for _ in range(stages)]
    act_in_flight = [0] * stages     # activations sent to stage s and not yet received
    grad_in_flight = [0] * stages
    for step in range(n):
        for s in range(stages):
            for c in gens[s][step]:
                nm = c.name
                if nm in ("SendActivation", "SendActivationRecvGrad"):
                    act_in_flight[s + 1] += 1
                if nm in ("SendGrad", "SendGradRecvActivation") and s > 0:
                    grad_in_flight[s - 1] += 1      # stage 0 emits no-op SendGrad in the 2-stage shifted case
        for s in range(stages):
            for c in gens[s][step]:
                nm = c.name
                if nm in ("RecvActivation", "SendGradRecvActivation"):
                    if s > 0:
                        act_in_flight[s] -= 1
                if nm in ("RecvGrad", "SendActivationRecvGrad", "RecomputeRecvGrad"):
                    grad_in_flight[s] -= 1
                if nm in ("ForwardPass", "PreCheckpointForwardPass"):
                    fwd[s].append(c.buffer_id)
                if nm == "BackwardPass":
                    bwd[s].append(c.buffer_id)
            assert len(bwd[s]) <= len(fwd[s])
    for s in range(stages):
        assert len(fwd[s]) == mbs and len(bwd[s]) == mbs, (name, s, fwd[s], bwd[s])
        assert act_in_flight[s] == 0 and grad_in_flight[s] == 0, (name, s, act_in_flight, grad_in_flight)


@pytest.mark.parametrize("name", ["1f1b", "ds_default", "pre_recompute_1f1b", "last_no_recompute_1f1b"])
@pytest.mark.parametrize("stages,mbs", [(1, 1), (1, 4), (2, 2), (2, 8), (3, 5), (4, 4), (4, 16), (8, 8), (8, 32)])
def test_schedule_invariants(name, stages, mbs):
    if name == "last_no_recompute_1f1b" and stages < 2:
        pytest.skip("needs two stages")
    _simulate(name, stages, mbs)


@pytest.mark.parametrize("stages,mbs", [(2, 4), (3, 6), (4, 4), (4, 8), (8, 8), (8, 16)])
def test_shifted_schedule_invariants(stages, mbs):
    _simulate("full_critical_path_1f1b", stages, mbs)


def test_shifted_requires_enough_micro_batches():
    with pytest.raises(ValueError):
        S.make_schedule("shifted_critical_path", 2, 2, 0)
    with pytest.raises(ValueError):
        S.make_schedule("nope", 2, 2, 0)
