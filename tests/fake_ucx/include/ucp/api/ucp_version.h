/* Version of the stand-in UCP library of the tests (see ucp.h beside this file). */
#ifndef FAKE_UCP_VERSION_H_
#define FAKE_UCP_VERSION_H_
#define UCP_API_MAJOR 1
#define UCP_API_MINOR 17
#endif
