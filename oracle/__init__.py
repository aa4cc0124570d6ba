"""CPU checkers for the neighbour-graph path (test infrastructure only).

``neighbor_oracle`` wraps the plain-C restatement of the reference's CUDA
semantics; ``reference_cpu`` loads the reference's own compiled CPU path from
``oracle/_ref``.  Only tests, the smoke check and the benchmark's CPU-baseline
leg import this package; the product package never does.
"""
