"""Keyed timers with the reference's keys and summary format (light_dist_gnn/dist_utils/timer.py:30-85).

`timing(key)` is wall clock, as in the reference.  `timing_cuda(key)` does NOT synchronise the device around the
region the way the reference does (timer.py:16-24; four host syncs per stage there): it records a pair of CUDA
events on the current stream and adds their elapsed time when a summary is asked for, so timing a region leaves
the broadcast/SpMM overlap intact.  On a CPU-only process it degrades to wall clock.
"""
import statistics
import time
from collections import defaultdict

import torch


class TimerCtx:
    def __init__(self, timer, key, cuda):
        self.timer, self.key, self.cuda = timer, key, cuda and torch.cuda.is_available()

    def __enter__(self):
        if self.cuda:
            self.begin = torch.cuda.Event(enable_timing=True)
            self.begin.record()
        else:
            self.t0 = time.time()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.timer.pending.append((self.key, self.begin, end))
            if len(self.timer.pending) >= self.timer.MAX_PENDING:       # a long run never holds more than this many event pairs
                self.timer.resolve()
        else:
            self.timer.duration_dict[self.key] += time.time() - self.t0
        self.timer.count_dict[self.key] += 1


class DistTimer:
    MAX_PENDING = 4096

    def __init__(self, env):
        self.env = env
        self.start_time_dict = {}
        self.duration_dict = defaultdict(float)
        self.count_dict = defaultdict(int)
        self.pending = []

    def resolve(self, synchronize=True):
        """Adds the elapsed time of the recorded event pairs to their keys.  The training loop calls it with
        synchronize=False right after it has read the loss (the device is idle then), so the list never grows."""
        if self.pending:
            if synchronize:
                torch.cuda.synchronize(self.env.device if self.env.device.type == 'cuda' else None)
            for key, begin, end in self.pending:
                self.duration_dict[key] += begin.elapsed_time(end) / 1000.0
            self.pending = []

    _resolve = resolve

    def timing(self, key):
        return TimerCtx(self, key, cuda=False)

    def timing_cuda(self, key):
        return TimerCtx(self, key, cuda=True)

    def start(self, key):
        self.start_time_dict[key] = time.time()
        return self.start_time_dict[key]

    def stop(self, key, *other_keys):
        d = time.time() - self.start_time_dict[key]
        for k in (key,) + tuple(key + '-' + sub for sub in other_keys):
            self.duration_dict[k] += d
            self.count_dict[k] += 1

    def summary(self):
        self._resolve()
        return '\ntimer summary:\n' + '\n'.join('%6.2fs %5d %s' % (self.duration_dict[k], self.count_dict[k], k) for k in self.duration_dict)

    def sync_duration_dicts(self):
        self._resolve()
        self.all_durations = self.env.all_gather_object(dict(self.duration_dict))

    def _stats(self):
        self.sync_duration_dicts()
        rows = {}
        for key in self.duration_dict:
            data = [d.get(key, 0.0) for d in self.all_durations]
            # the reference calls statistics.stdev, which raises with one rank (timer.py:52); report 0 instead
            rows[key] = (statistics.mean(data), statistics.stdev(data) if len(data) > 1 else 0.0, data)
        return rows

    def summary_all(self):
        rows = self._stats()
        return '\ntimer summary:\n' + '\n'.join('%6.2fs %6.2fs %5d %s' % (rows[k][0], rows[k][1], self.count_dict[k], k) for k in rows)

    def detail_all(self):
        rows = self._stats()
        return '\ntimer summary:\n' + '\n'.join(
            '%6.2fs %6.2fs %5d %s \ndetail: %s \n--------------' % (rows[k][0], rows[k][1], self.count_dict[k], k,
                                                                   ' '.join('%6.2f' % x for x in rows[k][2])) for k in rows)
