"""CPU oracle of the EXL3 projection path. Test infrastructure only; see t3_oracle.h."""
