"""CPU oracle of the continuous-batching step - TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
package.  The shipped library (macllm-infer_b200/) never does.
"""
