"""Device communicator for upstream vLLM's ``GroupCoordinator`` (see :mod:`.b200_communicator`)."""
