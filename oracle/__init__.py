"""TEST INFRASTRUCTURE: CPU oracle for the newt_b200 kernel library.

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may
import this package.  `oracle.cport` wraps the C restatement in
newt_oracle.c; `oracle.torch_ref` restates the torch calls the reference's own
tests and examples compare against.
"""
