"""Import-path alias: ``triton_dist.kernels.dcu.*`` resolves to the tridist_b200 operators, so that
scripts written against the reference library's module layout keep working."""
