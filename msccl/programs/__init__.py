"""MSCCLang programs shipped with the package (registered as plans by ``msccl.autosynth``)."""
