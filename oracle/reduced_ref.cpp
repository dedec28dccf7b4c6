extern "C" int oracle_reduced_placeholder(void){return 0;}
