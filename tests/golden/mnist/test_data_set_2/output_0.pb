
"(láÅ4‹Ä’†DMWÄ‘ÆDË¿Ä>á'ÅìaÂ¤&•B6hEBPlus214_Output_0