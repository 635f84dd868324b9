"""CPU oracle for the parity tests and the benchmark's CPU baseline.

Test infrastructure only: the product package never imports this.
"""
