"""CPU parity checker for rocwmma_b200.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference arm of bench.py may
import this package.  The product (rocwmma_b200/) never does.
"""
