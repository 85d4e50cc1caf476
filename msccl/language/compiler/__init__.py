"""MSCCLang compiler passes: fusion -> depth annotation -> channel/threadblock scheduling ->
dependency inference -> scratch placement -> replication -> static verification."""
