"""Python front-ends of the sm_100a kernels, each with an fp32 PyTorch oracle used by the tests."""
