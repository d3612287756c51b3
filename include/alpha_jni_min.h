/*
 * The part of the Java Native Interface that the JNI shim of this library uses, for building on a
 * machine without a JDK.  Types and function-table slots follow the JNI specification ("Interface
 * Function Table"): FindClass is slot 6, ThrowNew 14, GetArrayLength 171, GetLongArrayRegion 204,
 * ExceptionCheck 228.  Define ALPHA_USE_SYSTEM_JNI to build against the JDK's own <jni.h> instead;
 * the shim's source is the same for both.
 */
#ifndef ALPHA_JNI_MIN_H
#define ALPHA_JNI_MIN_H

#ifdef ALPHA_USE_SYSTEM_JNI
#include <jni.h>
#else

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t jint;
typedef int64_t jlong;
typedef uint8_t jboolean;
typedef jint jsize;

struct _jobject;
typedef struct _jobject* jobject;
typedef jobject jclass;
typedef jobject jarray;
typedef jarray jlongArray;

#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define ALPHA_JNI_SLOTS 235

struct JNINativeInterface_ {
    void* slot[ALPHA_JNI_SLOTS];
};

#ifdef __cplusplus
struct JNIEnv_ {
    const struct JNINativeInterface_* functions;

    jclass FindClass(const char* name)
    {
        typedef jclass (*fn)(JNIEnv_*, const char*);
        return reinterpret_cast<fn>(functions->slot[6])(this, name);
    }
    jint ThrowNew(jclass cls, const char* msg)
    {
        typedef jint (*fn)(JNIEnv_*, jclass, const char*);
        return reinterpret_cast<fn>(functions->slot[14])(this, cls, msg);
    }
    jsize GetArrayLength(jarray a)
    {
        typedef jsize (*fn)(JNIEnv_*, jarray);
        return reinterpret_cast<fn>(functions->slot[171])(this, a);
    }
    void GetLongArrayRegion(jlongArray a, jsize start, jsize len, jlong* buf)
    {
        typedef void (*fn)(JNIEnv_*, jlongArray, jsize, jsize, jlong*);
        reinterpret_cast<fn>(functions->slot[204])(this, a, start, len, buf);
    }
    jboolean ExceptionCheck()
    {
        typedef jboolean (*fn)(JNIEnv_*);
        return reinterpret_cast<fn>(functions->slot[228])(this);
    }
};
typedef JNIEnv_ JNIEnv;
#else
typedef const struct JNINativeInterface_* JNIEnv;
#endif

#ifdef __cplusplus
}
#endif
#endif /* ALPHA_USE_SYSTEM_JNI */
#endif /* ALPHA_JNI_MIN_H */
