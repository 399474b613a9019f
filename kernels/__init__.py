"""Import alias so code written against the reference's layout (`from kernels import kvskip`)
resolves to the sm_100a implementation in `kvskip_b200`."""
