"""CPU reference math: the oracle every GPU kernel and every distributed path is checked against."""
