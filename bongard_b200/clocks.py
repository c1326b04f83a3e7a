"""SM-clock record of a timed region: nvidia-smi sampled every 200 ms while it runs.

A timing without this record cannot be told apart from one taken on a throttled or
clock-locked GPU, so the benchmark and every op-level timing print it beside the number.
Only reads the GPU's state; never changes a setting.
"""

from __future__ import annotations

import os
import subprocess
import tempfile


class ClockSampler:
    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')
    REASONS = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')

    def __init__(self, index=0):
        self.index, self.proc, self.out = index, None, None
        self.path = os.path.join(tempfile.gettempdir(), f'bg_clocks_{os.getpid()}_{id(self):x}.csv')

    def start(self):
        try:
            self.out = open(self.path, 'w')
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '200'], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def stop(self):
        """{'sm_mhz': median, 'sm_max_mhz', 'power_w': median, 'samples', 'reasons': [...]}"""
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'samples': 0, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        self.proc.wait()
        self.out.close()
        sm, mx, power, reasons = [], [], [], set()
        with open(self.path) as lines:
            for line in lines:
                parts = [p.strip() for p in line.split(',')]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                    power.append(float(parts[2]))
                except ValueError:
                    continue
                for name, flag in zip(self.REASONS, parts[3:7]):
                    if flag.lower().startswith('active'):
                        reasons.add(name)
        os.unlink(self.path)
        sm.sort()
        power.sort()
        return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'power_w': power[len(power) // 2] if power else None, 'samples': len(sm), 'reasons': sorted(reasons)}

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        if self.proc is not None and self.proc.poll() is None:
            self.record = self.stop()
        return False
