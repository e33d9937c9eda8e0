"""CPU oracle for the fm scan path -- TEST INFRASTRUCTURE ONLY.

Nothing in the product package ``fm_b200`` imports this.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` do, and
only as the checker or the timed CPU baseline.

* ``oracle.c_oracle``   -- ctypes wrapper over ``fm_scan_oracle.c`` (fast, fp32 and fp64).
* ``oracle.torch_loop`` -- the reference's time-step loop restated with torch ops
  (``fm/scan/fm_pytorch.py:3-42``); it is the CPU implementation whose speed
  ``bench.py --impl reference`` reports.
"""
