"""Drop-in counterparts of the reference's TLX tutorial entry points
(``third_party/tlx/tutorials/*.py``): same function names and arguments, torch tensors in
and out, hand-written sm_100a kernels underneath."""
