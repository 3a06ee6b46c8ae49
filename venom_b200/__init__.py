"""venom_b200: a Blackwell (sm_100a) implementation of the V:N:M sparse x dense product (Spatha),
its dense->V:N:M compressor and an N-sharded multi-GPU launcher, behind a C ABI."""
