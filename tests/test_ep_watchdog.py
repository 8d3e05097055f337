"""Host watchdog of expert-parallel passes: the polling loop with scripted actions, no GPU and no NCCL.

The failure is made on the host: a communicator that reports an asynchronous error, a pass that never completes, a
pass that fails - the fakes of the three calls the loop makes (event query, async-error query, abort)."""
import time

import pytest

from dflb import pkg


def test_a_pass_that_completes_is_not_aborted():
    assert pkg.ep_watchdog_selftest(0, after_polls=5, timeout_ms=500) == 0


def test_an_asynchronous_communicator_error_aborts_and_reports_collective():
    with pytest.raises(pkg.DflError) as e:
        pkg.ep_watchdog_selftest(1, after_polls=4, timeout_ms=2000)
    assert e.value.name == "COLLECTIVE" and e.value.aborted == 1
    assert "asynchronous error (6)" in str(e.value)


def test_a_pass_that_never_completes_runs_into_the_limit():
    t0 = time.monotonic()
    with pytest.raises(pkg.DflError) as e:
        pkg.ep_watchdog_selftest(2, timeout_ms=150)
    dt = time.monotonic() - t0
    assert e.value.name == "COLLECTIVE" and e.value.aborted == 1
    assert "did not complete within 150 ms" in str(e.value)
    assert 0.14 <= dt < 2.0   # gave up at the limit, and the drain wait after the abort ended at once


def test_a_failed_pass_aborts_too():
    with pytest.raises(pkg.DflError) as e:
        pkg.ep_watchdog_selftest(3, after_polls=2, timeout_ms=500)
    assert e.value.name == "COLLECTIVE" and e.value.aborted == 1


def test_bad_arguments_are_refused():
    for args in ((4, 1, 100), (0, 1, 0), (0, 1, 20000)):
        with pytest.raises(pkg.DflError) as e:
            pkg.ep_watchdog_selftest(*args)
        assert e.value.name == "BAD_ARG"
