"""TEST INFRASTRUCTURE: CPU oracle of the broadcast-SpMM / GCN-epoch path.

Only tests, the smoke check and the benchmark's CPU-baseline / reference legs may import this
package.  Nothing in the product imports it, and the product raises when its CUDA library is absent
instead of falling back to anything here.
"""
