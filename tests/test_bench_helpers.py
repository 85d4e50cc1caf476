"""Host-side pieces of bench.py that need no GPU: bus-bandwidth factors, parsing of the clock samples, and the rule
that samples of the sustained region stand in when the short timed region yielded none."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location('bench_under_test', os.path.join(ROOT, 'bench.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_bus_factors_follow_nccl_tests():
    b = _bench()
    assert b.bus_factor(1) == 1.0 and b.bus_factor(8) == 1.75 and b.bus_factor(2) == 1.0
    assert b.bus_factor(8, 'allgather') == 0.875 and b.bus_factor(4, 'alltoall') == 0.75


def test_clock_samples_are_parsed_and_throttle_reasons_collected():
    b = _bench()

    class Done:
        def terminate(self):
            pass

    class Joined:
        def join(self, timeout=None):
            pass

    s = b.ClockSampler(0)
    s.proc, s.thread = Done(), Joined()
    s.rows = [['0', '1965', '1965', '412.5', '0x0', 'Not Active', 'Not Active', 'Not Active', 'Not Active'],
              ['0', '1305', '1965', '998.1', '0x4', 'Not Active', 'Not Active', 'Not Active', 'Active'],
              ['0', '1950', '1965', '640.0', '0x0', 'Not Active', 'Not Active', 'Not Active', 'Not Active'],
              ['garbage']]
    got = s.stop()
    assert got == {'sm_mhz': 1950.0, 'sm_max_mhz': 1965.0, 'reasons': ['sw_power_cap'], 'samples': 3}


def test_sustained_region_supplies_the_clock_record_when_the_timed_region_was_too_short():
    b = _bench()

    class Sampler:
        def __init__(self, index):
            pass

        def start(self):
            pass

        def stop(self):
            return {'sm_mhz': 1965.0, 'sm_max_mhz': 1965.0, 'reasons': [], 'samples': 40}

    b.ClockSampler = Sampler
    b._sustained = lambda n, ms, step, sync=None: {'steps': 440, 'ms_per_step': ms, 'timed_region_s': 1.1}
    empty = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
    sustained, clocks = b._sustained_sampled(0, empty, 8, 2.5, None)
    assert sustained['steps'] == 440 and clocks['samples'] == 40 and 'sustained region' in clocks['region']
    kept = {'sm_mhz': 1965.0, 'sm_max_mhz': 1965.0, 'reasons': [], 'samples': 3}
    assert b._sustained_sampled(0, kept, 8, 2.5, None, None)[1] is kept
