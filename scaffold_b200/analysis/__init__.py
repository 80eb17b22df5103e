"""Analysis tools that need no GPU: symbolic shape tracing of the U-Net, the convolution cost model,
the reference / tolerance policy of the kernel tests, and the census of convolutions a run issues."""
