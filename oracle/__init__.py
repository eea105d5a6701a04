"""CPU oracle for Tyr's attention path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm
may import this package; nothing under tyr_b200/ does.

Two checkers:
  * `c_oracle`   — ctypes binding of attn_oracle.c, the plain-C restatement.
  * `aten_path`  — the ATen operator the reference calls (cc/src/tyr.cpp:2578,
    3941, 4126), reached through Python torch on the CPU, with the reference's
    repeat_interleave GQA expansion restated around it.
Parity pin: attn_oracle.c is checked against committed outputs of the ATen
operator (tests/golden/) and closed-form cases; the reference's own tests hold no
golden vectors for this path.
"""
