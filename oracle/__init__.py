"""CPU restatement of the reference's sparse MLA numerical oracle.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this
directory. It is imported by the tests, by the smoke check and by the CPU
baseline / reference arm of the benchmark, always as the checker or the timed
CPU baseline, never as the implementation that serves a call.
"""
