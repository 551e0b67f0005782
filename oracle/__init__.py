"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference attention path.

Nothing in the shipped package may import this; it exists to check the CUDA path.
"""
