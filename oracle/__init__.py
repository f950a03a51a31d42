"""CPU oracle for the tile-sparse hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this directory is part of the product: only tests/, the smoke check and the CPU
baseline leg of the benchmark may import it, as the checker the CUDA path is compared against.
"""
