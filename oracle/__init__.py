"""CPU oracle for the linear-recurrence path -- TEST INFRASTRUCTURE, not product code.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import this package.  The product package (``philtorch_b200``) never does and has no
CPU fallback.

* ``oracle.cport``   -- ctypes front-end of ``recur_oracle.c`` (plain C restatement).
* ``oracle.refext``  -- loader for the reference project's own CPU extension, when it
  was compiled into ``oracle/_ref`` (see ``build_ref.py``), with the reference's
  adjoint rules restated on top of its forward ops.
* ``oracle.inputs``  -- seeded synthetic inputs for the five benchmark configurations.
"""
